"""The shared library loads without a GPU, exports every symbol the C header
declares and the reference's C++ symbols for the decode path, and the
reference's own consumers link against it unchanged (where their sources are
present)."""
import os
import re
import shutil
import subprocess

import pytest

from blackwell_b200 import _build, _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REFERENCE = os.environ.get("BW_REFERENCE_DIR", os.path.join(os.sep, "root", "reference"))

# Itanium-mangled names the reference's consumers reference (namespace blackwell::kernels).
DROPIN_SYMBOLS = [
    "_ZN9blackwell7kernels17gemv_int4_batchedEPfPKhPKfS3_S5_iiiP11CUstream_st",
    "_ZN9blackwell7kernels14gemv_int4_warpEPfPKvPKfS3_S5_iiP11CUstream_st",
    "_ZN9blackwell7kernels13quantize_int4EPvPfPKfiP11CUstream_st",
    "_ZN9blackwell7kernels21quantize_int4_batchedEPvPfPKfiiP11CUstream_st",
    "_ZN9blackwell7kernels13quantize_int8EPvPfPKfiP11CUstream_st",
    "_ZN9blackwell7kernels13fused_rmsnormEPfPKfS3_ifP11CUstream_st",
    "_ZN9blackwell7kernels21fused_rmsnorm_batchedEPfPKfS3_ifiP11CUstream_st",
    "_ZN9blackwell7kernels12apply_swigluEPfPKfS3_iP11CUstream_st",
    "_ZN9blackwell7kernels15vector_add_fp32EPfPKfS3_iP11CUstream_st",
    "_ZN9blackwell7kernels15update_kv_cacheEPfS1_PKfS3_iiiiiP11CUstream_st",
    "_ZN9blackwell7kernels22update_kv_cache_deviceEPfS1_PKfS3_iPKiiiiP11CUstream_st",
    "_ZN9blackwell7kernels28attention_decode_batched_gqaEPfPKfS3_S3_iiiiiimmP11CUstream_st",
    "_ZN9blackwell7kernels35attention_decode_batched_gqa_deviceEPfPKfS3_S3_PKiiiiiimmP11CUstream_st",
    "_ZN9blackwell7kernels24apply_repetition_penaltyEPfPKiifiP11CUstream_st",
    "_ZN9blackwell7kernels10sample_gpuEPKfifiPiyiP11CUstream_st",
    "_ZN9blackwell7kernels17sample_argmax_gpuEPKfiPiP11CUstream_st",
    "_ZN9blackwell7kernels17fused_rope_decodeEPfPKfS3_PKiiiiP11CUstream_st",
    "_ZN9blackwell7kernels24fused_rmsnorm_quant_int4EPhPfPKfS4_ifP11CUstream_st",
    "_ZN9blackwell7kernels23fused_swiglu_quant_int4EPhPfPKfS4_iP11CUstream_st",
]


@pytest.fixture(scope="module")
def so_path():
    if not os.path.exists(_lib.SO_PATH):
        _build.build()
    return _lib.SO_PATH


def test_library_loads_and_exports_every_declared_symbol(so_path):
    lib = _lib.load()
    names = _lib.declared_symbols()
    assert len(names) >= 30
    for n in names:
        assert hasattr(lib, n), n
    assert lib.bw_version() >= 100


def test_argument_checks_need_no_gpu(so_path):
    lib = _lib.load()
    # rejected before any CUDA call: bad K, null pointers
    assert lib.bw_gemv_int4_batched(None, None, None, None, None, 100, 16, 1, None) == 1
    assert lib.bw_quantize_int8(None, None, None, 15, None) == 1
    assert lib.bw_gemv_w4a8(None, None, None, None, None, 4096, 16, 0, None) == 1
    assert lib.bw_set_tuning(99, 0) == 1


def test_cxx_dropin_symbols_exported(so_path):
    out = subprocess.run(["nm", "-D", "--defined-only", so_path], capture_output=True, text=True, check=True).stdout
    have = set(l.split()[-1] for l in out.splitlines() if l.strip())
    missing = [s for s in DROPIN_SYMBOLS if s not in have]
    assert not missing, missing
    ar = os.path.join(os.path.dirname(so_path), "libblackwell_kernels.a")
    assert os.path.exists(ar)


def test_dropin_header_matches_c_header():
    """Every C++ forwarder has a C entry point of the same name."""
    hpp = open(os.path.join(ROOT, "include", "blackwell_b200_dropin.hpp")).read()
    cxx = set(re.findall(r"cudaError_t\s+([a-z0-9_]+)\s*\(", hpp))
    c = set(n[3:] for n in _lib.declared_symbols())
    assert cxx and cxx <= c, cxx - c


@pytest.mark.skipif(not os.path.isdir(REFERENCE) or shutil.which("nvcc") is None,
                    reason="reference sources or nvcc not present on this machine")
@pytest.mark.parametrize("consumer", ["server/inference_server_int4_batched.cu",
                                      "bench/text_generate_int4_batched.cu"])
def test_reference_consumers_link_unchanged(so_path, consumer, tmp_path):
    ar = os.path.join(os.path.dirname(so_path), "libblackwell_kernels.a")
    exe = tmp_path / "consumer"
    cmd = ["nvcc", "-std=c++17", "-O1", "-gencode", "arch=compute_100a,code=sm_100a", "-w",
           "-I", os.path.join(REFERENCE, "include"), os.path.join(REFERENCE, consumer), ar, "-o", str(exe)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    assert exe.exists()
