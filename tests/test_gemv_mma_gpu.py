"""The streaming kernel with warp-level tensor-core dots (mma.sync.m16n8k32.s8; 3 to 16 sequences per launch),
through the same C entry points as the other GEMV kernels, against the double-precision oracle: both scale types,
K processed in windows, scale rows that are not 16-byte multiples, ragged row counts, the fused prologues, and
bit-level agreement of the integer dots with the dp4a kernel."""
import numpy as np
import pytest

import oracle
from blackwell_b200 import synth
from tests.util import max_abs_rel, to_dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def k(cuda):
    """The kernels with the mma.sync kernel's range opened to 3..16 sequences (by default, routing by measurement
    gives it 5..16 and leaves multi-window shapes above 8 sequences to the tcgen05 kernel)."""
    from blackwell_b200 import kernels

    kernels.set_tuning(13, 3)
    yield kernels
    kernels.set_tuning(13, 0)


# (M, K, N): every M of the kernel's range; K = 10944 has binary16 scale rows of 1368 bytes (8 mod 16: the cp.async
# path); K = 25600 at M = 16 and K = 10944 at M >= 9 need activation windows; N not a multiple of the 32-row tile and
# smaller than one tile per SM.
W4A8_CASES = [(3, 4096, 4096), (4, 4096, 333), (5, 10944, 512), (6, 5120, 1000), (7, 4096, 6144), (8, 4096, 21888),
              (8, 10944, 300), (9, 4096, 4096), (12, 10944, 4096), (13, 1056, 77), (16, 4096, 5000), (16, 25600, 640),
              (16, 10944, 1024), (11, 64, 40), (16, 32, 9), (10, 2080, 31)]


@pytest.mark.parametrize("M,K,N", W4A8_CASES)
def test_mma_w4a8_matches_oracle(k, M, K, N):
    import torch

    W, sc16, _ = synth.int4_weights(N, K, seed=3 * M + K + N, full_range=True)
    x32 = synth.activations_f16(M, K, 1001).astype(np.float32) * 1.5
    xq, xs = oracle.quantize_int8(x32)
    y = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    k.gemv_w4a8(y, to_dev(xq), to_dev(xs), to_dev(W), to_dev(sc16.view(np.uint16)), K, N, M)
    torch.cuda.synchronize()
    assert k.device_status() == 0
    out = y.cpu().numpy()
    assert np.isfinite(out).all()
    assert max_abs_rel(out, oracle.gemv_w4a8_f64(xq, xs, W, sc16)) < 2e-5


@pytest.mark.parametrize("M,K,N", [(3, 4096, 1024), (9, 4096, 257), (16, 10944, 130), (16, 1024, 64), (14, 25600, 48)])
def test_mma_w4a4_fp32_scales_matches_oracle(k, M, K, N):
    """The reference's own format (INT4 activations, fp32 scales): gemv_int4_batched at 3..16 sequences."""
    import torch

    W, _, sc32 = synth.int4_weights(N, K, seed=M + K + N, full_range=True)
    x32 = synth.activations_f16(M, K, 1002).astype(np.float32)
    xq, xs = oracle.quantize_int4(x32)
    y = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    k.gemv_int4_batched(y, to_dev(xq), to_dev(xs), to_dev(W), to_dev(sc32), K, N, M)
    torch.cuda.synchronize()
    assert k.device_status() == 0
    assert max_abs_rel(y.cpu().numpy(), oracle.gemv_w4a4_f64(xq, xs, W, sc32)) < 2e-5


@pytest.mark.parametrize("slab,stages", [(32, 0), (16, 2), (64, 2)])
def test_mma_other_ring_shapes(k, slab, stages):
    import torch

    M, K, N = 12, 4096, 1500
    W, sc16, _ = synth.int4_weights(N, K, seed=1003)
    x16 = synth.activations_f16(M, K, 1004)
    xq, xs = oracle.quantize_int8(x16.astype(np.float32))
    y = torch.empty((M, N), dtype=torch.float32, device="cuda")
    k.set_tuning(12, slab)
    k.set_tuning(15, stages)
    try:
        k.gemv_w4a8_f16in(y, to_dev(x16.view(np.uint16)), to_dev(W), to_dev(sc16.view(np.uint16)), K, N, M)
        torch.cuda.synchronize()
    finally:
        k.set_tuning(12, 0)
        k.set_tuning(15, 0)
    assert k.device_status() == 0
    assert max_abs_rel(y.cpu().numpy(), oracle.gemv_w4a8_f64(xq, xs, W, sc16)) < 2e-5


def test_mma_fused_prologues_residual_and_determinism(k):
    import torch

    M, K, N = 11, 4096, 700
    W, sc16, _ = synth.int4_weights(N, K, seed=1005)
    x32 = synth.activations_f16(M, K, 1006).astype(np.float32)
    nw = synth.norm_weight(K, 1007)
    res = synth.activations_f16(M, N + 4, 1008).astype(np.float32)
    Wd, sd = to_dev(W), to_dev(sc16.view(np.uint16))
    y = to_dev(res.copy())
    k.gemv_w4a8_decode(y, N + 4, y, to_dev(x32), None, 0, to_dev(nw), 1e-6, Wd, sd, K, N, M)
    xq, xs = oracle.quantize_int8(oracle.rmsnorm(x32, nw))
    ref = res[:, :N] + oracle.gemv_w4a8_f64(xq, xs, W, sc16)
    out = y.cpu().numpy()
    assert max_abs_rel(out[:, :N], ref) < 1e-3
    assert np.array_equal(out[:, N:], res[:, N:])
    y2 = to_dev(res.copy())
    k.gemv_w4a8_decode(y2, N + 4, y2, to_dev(x32), None, 0, to_dev(nw), 1e-6, Wd, sd, K, N, M)
    assert torch.equal(y, y2)
    gu = synth.activations_f16(M, 2 * K, 1009).astype(np.float32)
    gud = to_dev(gu)
    y3 = torch.empty((M, N), dtype=torch.float32, device="cuda")
    k.gemv_w4a8_decode(y3, 0, None, gud, gud[:, K:], 2 * K, None, 0.0, Wd, sd, K, N, M)
    xq, xs = oracle.quantize_int8(oracle.swiglu(np.ascontiguousarray(gu[:, :K]), np.ascontiguousarray(gu[:, K:])))
    assert max_abs_rel(y3.cpu().numpy(), oracle.gemv_w4a8_f64(xq, xs, W, sc16)) < 1e-3
    assert k.device_status() == 0


def test_mma_windows_with_residual(k):
    """K in several activation windows: the first window writes y (plus the residual), the others add to it."""
    import torch

    M, K, N = 16, 10944, 500
    W, sc16, _ = synth.int4_weights(N, K, seed=1010)
    x32 = synth.activations_f16(M, K, 1011).astype(np.float32)
    res = synth.activations_f16(M, N, 1012).astype(np.float32)
    y = to_dev(res.copy())
    k.gemv_w4a8_decode(y, 0, y, to_dev(x32), None, 0, None, 0.0, to_dev(W), to_dev(sc16.view(np.uint16)), K, N, M)
    xq, xs = oracle.quantize_int8(x32)
    assert max_abs_rel(y.cpu().numpy(), res + oracle.gemv_w4a8_f64(xq, xs, W, sc16)) < 2e-5
    assert k.device_status() == 0


def test_mma_integer_dots_equal_the_dp4a_kernel_bitwise(k):
    """With all scales 1 the outputs are exact integers: the mma kernel (M = 16 and M = 5) and the dp4a kernel (the same
    sequences with the mma kernel switched off) must agree bit for bit, and with the oracle's per-block dots."""
    import torch

    K, N = 2048, 300
    W, _, _ = synth.int4_weights(N, K, seed=1013, full_range=True)
    ones16 = np.ones((N, K // 16), np.float16)
    xq = synth.rng(1014).integers(-127, 128, size=(16, K), dtype=np.int8)
    xs = np.full((16, K // 16), 16.0, np.float32)  # x_sc / 16 = 1
    Wd, sd = to_dev(W), to_dev(ones16.view(np.uint16))
    y16 = torch.empty((16, N), dtype=torch.float32, device="cuda")
    y5 = torch.empty((5, N), dtype=torch.float32, device="cuda")
    y5d = torch.empty((5, N), dtype=torch.float32, device="cuda")
    k.gemv_w4a8(y16, to_dev(xq), to_dev(xs), Wd, sd, K, N, 16)
    k.gemv_w4a8(y5, to_dev(xq[:5]), to_dev(xs[:5]), Wd, sd, K, N, 5)
    k.set_tuning(13, 99)   # smallest batch of the mma kernel: beyond its range = off
    try:
        k.gemv_w4a8(y5d, to_dev(xq[:5]), to_dev(xs[:5]), Wd, sd, K, N, 5)
    finally:
        k.set_tuning(13, 0)
    assert torch.equal(y16[:5], y5) and torch.equal(y5, y5d)
    # up to 4 sequences take the packed form (both k-blocks of a column in one MMA); it can also be switched off
    y4 = torch.empty((4, N), dtype=torch.float32, device="cuda")
    y4u = torch.empty((4, N), dtype=torch.float32, device="cuda")
    k.gemv_w4a8(y4, to_dev(xq[:4]), to_dev(xs[:4]), Wd, sd, K, N, 4)
    k.set_tuning(18, 0)
    try:
        k.gemv_w4a8(y4u, to_dev(xq[:4]), to_dev(xs[:4]), Wd, sd, K, N, 4)
    finally:
        k.set_tuning(18, 1)
    assert torch.equal(y4, y16[:4]) and torch.equal(y4u, y16[:4])
    dots = oracle.block_dots_w4a8(W, xq[3]).sum(-1) * 16
    assert np.array_equal(y16[3].cpu().numpy(), dots.astype(np.float32))
