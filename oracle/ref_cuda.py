"""The reference's own CUDA kernels, rebuilt unchanged for sm_100a -- TEST INFRASTRUCTURE ONLY.

``make -C oracle ref`` compiles the reference's decode-path translation units
where they lie into ``oracle/_ref/libblackwell_ref.so``.  This module binds the
C++ symbols of that library (Itanium-mangled names of ``blackwell::kernels::*``)
with ctypes so that GPU tests and the benchmark can run the reference kernels
on the same device buffers as ours: they pin the CPU oracle and serve as the
"kernel to beat".  Nothing in the shipped package imports this module.

Known limits of the reference kernels (not comparators outside them):
M <= 16 and N % 16 == 0 for the GEMV, RMSNorm H <= 4096, attention context
<= 3968 positions and a race in its softmax for longer contexts.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
SO_PATH = os.path.join(_HERE, "_ref", "libblackwell_ref.so")

_NS = "_ZN9blackwell7kernels"
_SYMS = {
    "gemv_int4_batched": _NS + "17gemv_int4_batchedEPfPKhPKfS3_S5_iiiP11CUstream_st",
    "gemv_int4_warp": _NS + "14gemv_int4_warpEPfPKvPKfS3_S5_iiP11CUstream_st",
    "quantize_int4": _NS + "13quantize_int4EPvPfPKfiP11CUstream_st",
    "quantize_int4_batched": _NS + "21quantize_int4_batchedEPvPfPKfiiP11CUstream_st",
    "quantize_int8": _NS + "13quantize_int8EPvPfPKfiP11CUstream_st",
    "fused_rmsnorm": _NS + "13fused_rmsnormEPfPKfS3_ifP11CUstream_st",
    "fused_rmsnorm_batched": _NS + "21fused_rmsnorm_batchedEPfPKfS3_ifiP11CUstream_st",
    "apply_swiglu": _NS + "12apply_swigluEPfPKfS3_iP11CUstream_st",
    "vector_add_fp32": _NS + "15vector_add_fp32EPfPKfS3_iP11CUstream_st",
    "update_kv_cache": _NS + "15update_kv_cacheEPfS1_PKfS3_iiiiiP11CUstream_st",
    "attention_decode_batched_gqa": _NS + "28attention_decode_batched_gqaEPfPKfS3_S3_iiiiiimmP11CUstream_st",
    "sample_argmax_gpu": _NS + "17sample_argmax_gpuEPKfiPiP11CUstream_st",
    "apply_repetition_penalty": _NS + "24apply_repetition_penaltyEPfPKiifiP11CUstream_st",
    "fused_rmsnorm_quant_int4": _NS + "24fused_rmsnorm_quant_int4EPhPfPKfS4_ifP11CUstream_st",
    "fused_swiglu_quant_int4": _NS + "23fused_swiglu_quant_int4EPhPfPKfS4_iP11CUstream_st",
}

_lib = None


def available() -> bool:
    return os.path.exists(SO_PATH)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(SO_PATH)
    return _lib


def _fn(name):
    return getattr(lib(), _SYMS[name])


def _p(t):
    return C.c_void_p(0 if t is None else t.data_ptr())


def _s(stream):
    import torch

    return C.c_void_p((stream or torch.cuda.current_stream()).cuda_stream)


def _chk(name, code):
    if code != 0:
        raise RuntimeError(f"reference {name} returned cudaError {code}")


def gemv_int4_batched(y, x_packed, x_scale, W_packed, W_scale, K, N, M, stream=None):
    _chk("gemv_int4_batched", _fn("gemv_int4_batched")(_p(y), _p(x_packed), _p(x_scale), _p(W_packed), _p(W_scale),
                                                       K, N, M, _s(stream)))


def gemv_int4_warp(y, x_packed, x_scale, W_packed, W_scale, K, N, stream=None):
    _chk("gemv_int4_warp", _fn("gemv_int4_warp")(_p(y), _p(x_packed), _p(x_scale), _p(W_packed), _p(W_scale), K, N,
                                                 _s(stream)))


def quantize_int4(out, sc, x, K, stream=None):
    _chk("quantize_int4", _fn("quantize_int4")(_p(out), _p(sc), _p(x), K, _s(stream)))


def quantize_int4_batched(out, sc, x, K, M, stream=None):
    _chk("quantize_int4_batched", _fn("quantize_int4_batched")(_p(out), _p(sc), _p(x), K, M, _s(stream)))


def quantize_int8(out, sc, x, n, stream=None):
    _chk("quantize_int8", _fn("quantize_int8")(_p(out), _p(sc), _p(x), n, _s(stream)))


def fused_rmsnorm(out, inp, w, n, eps, stream=None):
    _chk("fused_rmsnorm", _fn("fused_rmsnorm")(_p(out), _p(inp), _p(w), n, C.c_float(eps), _s(stream)))


def fused_rmsnorm_batched(out, inp, w, H, eps, M, stream=None):
    _chk("fused_rmsnorm_batched", _fn("fused_rmsnorm_batched")(_p(out), _p(inp), _p(w), H, C.c_float(eps), M,
                                                               _s(stream)))


def apply_swiglu(out, g, u, n, stream=None):
    _chk("apply_swiglu", _fn("apply_swiglu")(_p(out), _p(g), _p(u), n, _s(stream)))


def vector_add_fp32(out, a, b, n, stream=None):
    _chk("vector_add_fp32", _fn("vector_add_fp32")(_p(out), _p(a), _p(b), n, _s(stream)))


def update_kv_cache(kc, vc, k_new, v_new, batch_idx, seq_pos, nh, hd, max_seq, stream=None):
    _chk("update_kv_cache", _fn("update_kv_cache")(_p(kc), _p(vc), _p(k_new), _p(v_new), batch_idx, seq_pos, nh, hd,
                                                   max_seq, _s(stream)))


def attention_decode_batched_gqa(out, Q, Kc, Vc, seq_pos, nqh, nkv, hd, max_seq, M, kv_batch_elems, kv_layer_elems,
                                 stream=None):
    _chk("attention_decode_batched_gqa", _fn("attention_decode_batched_gqa")(
        _p(out), _p(Q), _p(Kc), _p(Vc), seq_pos, nqh, nkv, hd, max_seq, M, C.c_size_t(kv_batch_elems),
        C.c_size_t(kv_layer_elems), _s(stream)))


def sample_argmax_gpu(logits, vocab, out_id, stream=None):
    _chk("sample_argmax_gpu", _fn("sample_argmax_gpu")(_p(logits), vocab, _p(out_id), _s(stream)))


def apply_repetition_penalty(logits, recent, n, penalty, vocab, stream=None):
    _chk("apply_repetition_penalty", _fn("apply_repetition_penalty")(_p(logits), _p(recent), n, C.c_float(penalty),
                                                                     vocab, _s(stream)))


def fused_rmsnorm_quant_int4(out, sc, x, w, N, eps, stream=None):
    _chk("fused_rmsnorm_quant_int4", _fn("fused_rmsnorm_quant_int4")(_p(out), _p(sc), _p(x), _p(w), N,
                                                                     C.c_float(eps), _s(stream)))


def fused_swiglu_quant_int4(out, sc, g, u, N, stream=None):
    _chk("fused_swiglu_quant_int4", _fn("fused_swiglu_quant_int4")(_p(out), _p(sc), _p(g), _p(u), N, _s(stream)))
