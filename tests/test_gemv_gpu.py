"""Parity of the sm_100a INT4 GEMV kernels, called through the C ABI, against
the CPU oracle and against the reference's own CUDA kernel rebuilt for the box.

Bars: per-block int32 dot products bit-exact; fp32 outputs within max-abs-rel
1e-3 of the high-precision oracle (and of the reference kernel)."""
import numpy as np
import pytest

import oracle
from blackwell_b200 import synth
from tests.util import TOL, max_abs_rel, to_dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def k(cuda):
    from blackwell_b200 import kernels

    return kernels


def _run_w4a4(k, M, K, N, seed, x32=None, full_range=True):
    import torch

    W, sc16, sc32 = synth.int4_weights(N, K, seed, full_range=full_range)
    if x32 is None:
        x32 = synth.activations_f16(M, K, seed + 1).astype(np.float32)
    xq, xs = oracle.quantize_int4(x32)
    y = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    k.gemv_int4_batched(y, to_dev(xq), to_dev(xs), to_dev(W), to_dev(sc32), K, N, M)
    torch.cuda.synchronize()
    return y.cpu().numpy(), (xq, xs, W, sc16, sc32)


# (M, K, N): config-0 shape, odd block counts, ragged N, every M up to 17, multi-pass K
W4A4_CASES = [
    (1, 4096, 4096), (1, 4096, 1024), (2, 4096, 6144), (1, 10944, 512), (3, 10944, 130), (8, 4096, 257),
    (1, 16, 1), (1, 48, 7), (2, 1040, 33), (5, 2736, 64), (4, 5120, 96), (1, 25600, 40), (8, 25600, 24),
    (9, 512, 40), (16, 1024, 64), (17, 256, 19), (7, 8192, 300), (6, 4128, 50),
]


@pytest.mark.parametrize("M,K,N", W4A4_CASES)
def test_w4a4_matches_oracle(k, M, K, N):
    y, (xq, xs, W, _, sc32) = _run_w4a4(k, M, K, N, seed=M * 7 + K + N)
    ref = oracle.gemv_w4a4_f64(xq, xs, W, sc32)
    assert np.isfinite(y).all()
    assert max_abs_rel(y, ref) < TOL
    # fp32 accumulation should in fact be far tighter than the stated tolerance
    assert max_abs_rel(y, ref) < 2e-5
    assert k.device_status() == 0


@pytest.mark.parametrize("M,K,N", [(1, 4096, 4096), (4, 4096, 1024), (16, 1024, 64), (2, 10944, 4096)])
def test_w4a4_matches_reference_cuda_kernel(k, M, K, N):
    import torch

    from oracle import ref_cuda

    if not ref_cuda.available():
        pytest.fail("oracle/_ref/libblackwell_ref.so missing: run `make -C oracle ref` before shipping to the GPU box")
    y, (xq, xs, W, _, sc32) = _run_w4a4(k, M, K, N, seed=11)
    yr = torch.empty((M, N), dtype=torch.float32, device="cuda")
    ref_cuda.gemv_int4_batched(yr, to_dev(xq), to_dev(xs), to_dev(W), to_dev(sc32), K, N, M)
    torch.cuda.synchronize()
    yr = yr.cpu().numpy()
    assert max_abs_rel(y, yr) < TOL
    # and the exact-order oracle reproduces the reference kernel bit for bit
    assert np.array_equal(yr, oracle.gemv_w4a4_exact(xq, xs, W, sc32))


def test_gemv_int4_warp_is_the_m1_case(k):
    import torch

    M, K, N = 1, 4096, 777
    W, _, sc32 = synth.int4_weights(N, K, 5)
    x32 = synth.activations_f16(M, K, 6).astype(np.float32)
    xq, xs = oracle.quantize_int4(x32)
    y = torch.empty((N,), dtype=torch.float32, device="cuda")
    k.gemv_int4_warp(y, to_dev(xq[0]), to_dev(xs[0]), to_dev(W), to_dev(sc32), K, N)
    assert max_abs_rel(y.cpu().numpy(), oracle.gemv_w4a4_f64(xq, xs, W, sc32)[0]) < 2e-5


@pytest.mark.parametrize("a8", [0, 1])
@pytest.mark.parametrize("K,N", [(4096, 256), (1040, 37), (10944, 64)])
def test_block_dots_bit_exact(k, a8, K, N):
    import torch

    W, _, _ = synth.int4_weights(N, K, 21, full_range=True)
    x32 = synth.activations_f16(1, K, 22).astype(np.float32) * 3.0  # exercises the clamps
    if a8:
        xq, _ = oracle.quantize_int8(x32)
        ref = oracle.block_dots_w4a8(W, xq[0])
    else:
        xq, _ = oracle.quantize_int4(x32)
        ref = oracle.block_dots_w4a4(W, xq[0])
    dots = torch.empty((N, K // 16), dtype=torch.int32, device="cuda")
    k.gemv_block_dots(dots, to_dev(xq[0]), a8, to_dev(W), K, N)
    assert np.array_equal(dots.cpu().numpy(), ref)


def test_extreme_nibbles_and_scales(k):
    """All weights -8 against all activations -8 / +7, and the 127 clamp of the int8 path."""
    import torch

    K, N, M = 4096, 64, 2
    W = np.zeros((N, K // 2), np.uint8)  # nibble 0 everywhere = -8
    sc32 = np.full((N, K // 16), 0.5, np.float32)
    xq = np.zeros((M, K // 2), np.uint8)
    xq[1] = 0xFF  # +7
    xs = np.full((M, K // 16), 2.0, np.float32)
    y = torch.empty((M, N), dtype=torch.float32, device="cuda")
    k.gemv_int4_batched(y, to_dev(xq), to_dev(xs), to_dev(W), to_dev(sc32), K, N, M)
    y = y.cpu().numpy()
    assert np.all(y[0] == 64.0 * K) and np.all(y[1] == -56.0 * K)
    x8 = np.full((M, K), -127, np.int8)
    x8[1] = 127
    sc16 = np.full((N, K // 16), 0.5, np.float16)
    k.gemv_w4a8(y_t := torch.empty((M, N), dtype=torch.float32, device="cuda"), to_dev(x8), to_dev(xs), to_dev(W),
                to_dev(sc16.view(np.uint16)), K, N, M)
    y = y_t.cpu().numpy()
    assert np.all(y[0] == 8.0 * 127 * K) and np.all(y[1] == -8.0 * 127 * K)


W4A8_CASES = [(1, 4096, 4096), (1, 4096, 6144), (1, 10944, 4096), (2, 4096, 21888), (4, 4096, 1000), (8, 10944, 512),
              (3, 1040, 33), (1, 48, 5), (12, 2048, 100), (1, 5120, 640), (1, 25600, 64), (8, 8192, 96)]


@pytest.mark.parametrize("M,K,N", W4A8_CASES)
def test_w4a8_matches_oracle(k, M, K, N):
    import torch

    W, sc16, _ = synth.int4_weights(N, K, seed=K + N + M)
    x32 = synth.activations_f16(M, K, 31).astype(np.float32)
    xq, xs = oracle.quantize_int8(x32)
    y = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    k.gemv_w4a8(y, to_dev(xq), to_dev(xs), to_dev(W), to_dev(sc16.view(np.uint16)), K, N, M)
    ref = oracle.gemv_w4a8_f64(xq, xs, W, sc16)
    assert max_abs_rel(y.cpu().numpy(), ref) < 2e-5
    assert k.device_status() == 0


@pytest.mark.parametrize("M,K,N", [(1, 4096, 4096), (2, 10944, 512), (8, 4096, 300), (1, 5120, 1280)])
def test_w4a8_fused_f16_quantize_is_bit_identical_to_unfused(k, M, K, N):
    """The fused prologue quantizes with the same code as the stand-alone quantizer, so the two paths agree
    bit for bit, and both agree with the oracle's quantize + dequant-dot."""
    import torch

    W, sc16, _ = synth.int4_weights(N, K, seed=41)
    x16 = synth.activations_f16(M, K, 42)
    x16[0, :16] = 0
    xq, xs = oracle.quantize_int8(x16.astype(np.float32))
    Wd, sd = to_dev(W), to_dev(sc16.view(np.uint16))
    y_f = torch.empty((M, N), dtype=torch.float32, device="cuda")
    k.gemv_w4a8_f16in(y_f, to_dev(x16.view(np.uint16)), Wd, sd, K, N, M)
    y_u = torch.empty((M, N), dtype=torch.float32, device="cuda")
    k.gemv_w4a8(y_u, to_dev(xq), to_dev(xs), Wd, sd, K, N, M)
    assert torch.equal(y_f, y_u)
    assert max_abs_rel(y_f.cpu().numpy(), oracle.gemv_w4a8_f64(xq, xs, W, sc16)) < 2e-5


@pytest.mark.parametrize("M,K,N", [(1, 4096, 512), (4, 4096, 256), (2, 5120, 128), (1, 10944, 96)])
def test_w4a8_fused_rmsnorm_and_swiglu(k, M, K, N):
    """Fused RMSNorm (or SwiGLU) + quantize + GEMV against the unfused chain run on the same device: the
    normalised values differ from a CPU restatement in the last bit (rsqrtf, reduction order), so the
    comparison that must hold to 1e-3 is against the oracle chain, and the device chain must be close to
    the fused kernel to far better than that."""
    import torch

    W, sc16, _ = synth.int4_weights(N, K, seed=51)
    x32 = synth.activations_f16(M, K, 52).astype(np.float32)
    up = synth.activations_f16(M, K, 53).astype(np.float32)
    nw = synth.norm_weight(K, 54)
    Wd, sd = to_dev(W), to_dev(sc16.view(np.uint16))
    y = torch.empty((M, N), dtype=torch.float32, device="cuda")
    k.gemv_w4a8_f32in(y, to_dev(x32), to_dev(nw), 1e-6, Wd, sd, K, N, M)
    xn = oracle.rmsnorm(x32, nw)
    xq, xs = oracle.quantize_int8(xn)
    assert max_abs_rel(y.cpu().numpy(), oracle.gemv_w4a8_f64(xq, xs, W, sc16)) < TOL
    # no norm: plain f32 input
    k.gemv_w4a8_f32in(y, to_dev(x32), None, 0.0, Wd, sd, K, N, M)
    xq, xs = oracle.quantize_int8(x32)
    assert max_abs_rel(y.cpu().numpy(), oracle.gemv_w4a8_f64(xq, xs, W, sc16)) < 2e-5
    # swiglu prologue
    k.gemv_w4a8_swiglu(y, to_dev(x32), to_dev(up), Wd, sd, K, N, M)
    act = oracle.swiglu(x32, up)
    xq, xs = oracle.quantize_int8(act)
    assert max_abs_rel(y.cpu().numpy(), oracle.gemv_w4a8_f64(xq, xs, W, sc16)) < TOL


@pytest.mark.parametrize("M,K,N", [(1, 4096, 512), (3, 4096, 100)])
def test_int4_fused_prologues(k, M, K, N):
    import torch

    W, _, sc32 = synth.int4_weights(N, K, seed=61)
    x32 = synth.activations_f16(M, K, 62).astype(np.float32)
    up = synth.activations_f16(M, K, 63).astype(np.float32)
    nw = synth.norm_weight(K, 64)
    Wd, sd = to_dev(W), to_dev(sc32)
    y = torch.empty((M, N), dtype=torch.float32, device="cuda")
    k.gemv_int4_fused(y, to_dev(x32), None, None, 0.0, Wd, sd, K, N, M)
    xq, xs = oracle.quantize_int4(x32)
    assert max_abs_rel(y.cpu().numpy(), oracle.gemv_w4a4_f64(xq, xs, W, sc32)) < 2e-5
    k.gemv_int4_fused(y, to_dev(x32), None, to_dev(nw), 1e-6, Wd, sd, K, N, M)
    xq, xs = oracle.quantize_int4(oracle.rmsnorm(x32, nw))
    assert max_abs_rel(y.cpu().numpy(), oracle.gemv_w4a4_f64(xq, xs, W, sc32)) < 5e-3  # int4 ties flip whole steps
    k.gemv_int4_fused(y, to_dev(x32), to_dev(up), None, 0.0, Wd, sd, K, N, M)
    xq, xs = oracle.quantize_int4(oracle.swiglu(x32, up))
    assert max_abs_rel(y.cpu().numpy(), oracle.gemv_w4a4_f64(xq, xs, W, sc32)) < 5e-3


def test_plain_load_kernel_and_unaligned_operands(k):
    """Operands offset by 8 bytes (legal for the reference) take the plain-load kernel; forcing that kernel on
    an aligned problem gives the same result as the streaming kernel to fp32 rounding."""
    import torch

    M, K, N = 2, 4096, 200
    W, _, sc32 = synth.int4_weights(N, K, 71)
    x32 = synth.activations_f16(M, K, 72).astype(np.float32)
    xq, xs = oracle.quantize_int4(x32)
    ref = oracle.gemv_w4a4_f64(xq, xs, W, sc32)
    buf = torch.zeros(W.size + 8, dtype=torch.uint8, device="cuda")
    buf[8:] = to_dev(W).reshape(-1)
    y = torch.empty((M, N), dtype=torch.float32, device="cuda")
    k.gemv_int4_batched(y, to_dev(xq), to_dev(xs), buf[8:], to_dev(sc32), K, N, M)
    assert max_abs_rel(y.cpu().numpy(), ref) < 2e-5
    k.set_tuning(2, 1)
    try:
        y2 = torch.empty((M, N), dtype=torch.float32, device="cuda")
        k.gemv_int4_batched(y2, to_dev(xq), to_dev(xs), to_dev(W), to_dev(sc32), K, N, M)
    finally:
        k.set_tuning(2, 0)
    assert max_abs_rel(y2.cpu().numpy(), ref) < 2e-5


def test_argument_errors_match_reference_convention(k):
    import torch

    from blackwell_b200.kernels import CUDA_ERROR_INVALID_VALUE, KernelError

    t = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    f = torch.zeros(4096, dtype=torch.float32, device="cuda")
    for bad in [dict(K=24, N=16, M=1), dict(K=4096, N=0, M=1), dict(K=4096, N=16, M=0)]:
        with pytest.raises(KernelError) as e:
            k.gemv_int4_batched(f, t, f, t, f, bad["K"], bad["N"], bad["M"])
        assert e.value.code == CUDA_ERROR_INVALID_VALUE


def test_linearity_and_determinism_at_full_size(k):
    """Size-independent properties on the LM-head shape (too large for the CPU oracle in seconds):
    running twice gives identical bits; scaling every activation scale by 2 doubles y exactly; a row
    subset computed as its own GEMV equals the same rows of the full result."""
    import torch

    K, N, M = 4096, 151643, 1
    W, sc = synth.int4_weights_device(N, K, 81)
    x16 = synth.activations_f16_device(M, K, 82)
    xq = torch.empty((M, K), dtype=torch.int8, device="cuda")
    xs = torch.empty((M, K // 16), dtype=torch.float32, device="cuda")
    k.quantize_int8_f16(xq, xs, x16, M * K)
    y1 = torch.empty((M, N), dtype=torch.float32, device="cuda")
    y2 = torch.empty_like(y1)
    k.gemv_w4a8(y1, xq, xs, W, sc, K, N, M)
    k.gemv_w4a8(y2, xq, xs, W, sc, K, N, M)
    assert torch.equal(y1, y2)
    k.gemv_w4a8(y2, xq, xs * 2, W, sc, K, N, M)
    assert torch.equal(y2, y1 * 2)
    r0, r1 = 100000, 100512
    ys = torch.empty((M, r1 - r0), dtype=torch.float32, device="cuda")
    k.gemv_w4a8(ys, xq, xs, W[r0:r1], sc[r0:r1], K, r1 - r0, M)
    assert torch.equal(ys, y1[:, r0:r1])
    # a CPU spot check of 64 rows
    rows = slice(151579, 151643)
    ref = oracle.gemv_w4a8_f64(xq.cpu().numpy(), xs.cpu().numpy(), W[rows].cpu().numpy(),
                               sc[rows].cpu().numpy().view(np.uint16))
    assert max_abs_rel(y1[:, rows].cpu().numpy(), ref) < 2e-5
    assert k.device_status() == 0


def test_huge_k_scale_rows_not_16_byte_multiples(k):
    """K so large that only one row fits a tile, with binary16 scale rows of 8196 bytes: tiles would start at rows whose
    scales are not 16-byte aligned in global memory, which a bulk copy cannot fetch -- the planner must hand such a
    shape to the plain-load kernel (it once planned one-row tiles for it)."""
    import torch

    M, K, N = 1, 65568, 12
    W, sc16, _ = synth.int4_weights(N, K, 77)
    x32 = synth.activations_f16(M, K, 78).astype(np.float32)
    x8, x8s = oracle.quantize_int8(x32)
    y = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    k.gemv_w4a8(y, to_dev(x8), to_dev(x8s), to_dev(W), to_dev(sc16), K, N, M)
    torch.cuda.synchronize()
    assert max_abs_rel(y.cpu().numpy(), oracle.gemv_w4a8_f64(x8, x8s, W, sc16)) < 2e-5
    assert k.device_status() == 0
