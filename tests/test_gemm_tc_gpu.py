"""The tensor-core (tcgen05 kind::i8) path of the INT4 GEMV family, 9 to 64 sequences per launch and more in
passes, through the same C entry points as the small-batch kernel, against the double-precision oracle."""
import numpy as np
import pytest

import oracle
from blackwell_b200 import synth
from tests.util import max_abs_rel, to_dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def k(cuda):
    """The kernels with the mma.sync kernel switched off, so that every batch from 8 sequences up takes the tcgen05
    kernel as it does by default above 16."""
    from blackwell_b200 import kernels

    kernels.set_tuning(13, 99)
    yield kernels
    kernels.set_tuning(13, 0)


CASES = [(16, 256, 128), (9, 4096, 128), (16, 4096, 300), (17, 512, 129), (32, 4096, 1024), (33, 2048, 640),
         (64, 4096, 4096), (64, 10944, 512), (48, 5120, 1280), (65, 1024, 256), (100, 256, 130), (12, 288, 64)]


@pytest.mark.parametrize("M,K,N", CASES)
def test_tc_w4a8_prequantized(k, M, K, N):
    import torch

    W, sc16, _ = synth.int4_weights(N, K, seed=M + K + N, full_range=True)
    x32 = synth.activations_f16(M, K, 901).astype(np.float32) * 2.0
    xq, xs = oracle.quantize_int8(x32)
    y = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    k.gemv_w4a8(y, to_dev(xq), to_dev(xs), to_dev(W), to_dev(sc16.view(np.uint16)), K, N, M)
    torch.cuda.synchronize()
    assert k.device_status() == 0
    ref = oracle.gemv_w4a8_f64(xq, xs, W, sc16)
    out = y.cpu().numpy()
    assert np.isfinite(out).all()
    assert max_abs_rel(out, ref) < 2e-5


@pytest.mark.parametrize("ksplit", [1, 2, 5])
def test_tc_k_split_is_deterministic_and_exact_sum(k, ksplit):
    import torch

    M, K, N = 24, 4096, 384
    W, sc16, _ = synth.int4_weights(N, K, seed=77)
    x16 = synth.activations_f16(M, K, 902)
    xq, xs = oracle.quantize_int8(x16.astype(np.float32))
    Wd, sd, xd = to_dev(W), to_dev(sc16.view(np.uint16)), to_dev(x16.view(np.uint16))
    k.set_tuning(6, ksplit)
    try:
        y1 = torch.empty((M, N), dtype=torch.float32, device="cuda")
        y2 = torch.empty_like(y1)
        k.gemv_w4a8_f16in(y1, xd, Wd, sd, K, N, M)
        k.gemv_w4a8_f16in(y2, xd, Wd, sd, K, N, M)
    finally:
        k.set_tuning(6, 0)
    assert torch.equal(y1, y2)
    assert max_abs_rel(y1.cpu().numpy(), oracle.gemv_w4a8_f64(xq, xs, W, sc16)) < 2e-5
    assert k.device_status() == 0


def test_tc_fused_prologues_and_residual(k):
    import torch

    M, K, N = 20, 4096, 256
    W, sc16, _ = synth.int4_weights(N, K, seed=78)
    x32 = synth.activations_f16(M, K, 903).astype(np.float32)
    nw = synth.norm_weight(K, 904)
    res = synth.activations_f16(M, N, 905).astype(np.float32)
    Wd, sd = to_dev(W), to_dev(sc16.view(np.uint16))
    y = to_dev(res.copy())
    k.gemv_w4a8_decode(y, 0, y, to_dev(x32), None, 0, to_dev(nw), 1e-6, Wd, sd, K, N, M)
    xq, xs = oracle.quantize_int8(oracle.rmsnorm(x32, nw))
    ref = res + oracle.gemv_w4a8_f64(xq, xs, W, sc16)
    assert max_abs_rel(y.cpu().numpy(), ref) < 1e-3
    gu = synth.activations_f16(M, 2 * K, 906).astype(np.float32)
    gud = to_dev(gu)
    y2 = torch.empty((M, N), dtype=torch.float32, device="cuda")
    k.gemv_w4a8_decode(y2, 0, None, gud, gud[:, K:], 2 * K, None, 0.0, Wd, sd, K, N, M)
    act = oracle.swiglu(np.ascontiguousarray(gu[:, :K]), np.ascontiguousarray(gu[:, K:]))
    xq, xs = oracle.quantize_int8(act)
    assert max_abs_rel(y2.cpu().numpy(), oracle.gemv_w4a8_f64(xq, xs, W, sc16)) < 1e-3
    assert k.device_status() == 0


def test_tc_matches_small_batch_kernel_bitwise_dots(k):
    """Same integer dot products either way: with all scales 1 the outputs are exact integers and the dp4a
    kernel (M = 7) and the tensor-core kernel (M = 16, first 7 sequences) must agree exactly."""
    import torch

    K, N = 1024, 256
    W, _, _ = synth.int4_weights(N, K, seed=79, full_range=True)
    ones16 = np.ones((N, K // 16), np.float16)
    xq = synth.rng(907).integers(-127, 128, size=(16, K), dtype=np.int8)
    xs = np.full((16, K // 16), 16.0, np.float32)  # x_sc / 16 = 1
    Wd, sd = to_dev(W), to_dev(ones16.view(np.uint16))
    y16 = torch.empty((16, N), dtype=torch.float32, device="cuda")
    y7 = torch.empty((7, N), dtype=torch.float32, device="cuda")
    k.gemv_w4a8(y16, to_dev(xq), to_dev(xs), Wd, sd, K, N, 16)
    k.gemv_w4a8(y7, to_dev(xq[:7]), to_dev(xs[:7]), Wd, sd, K, N, 7)
    assert torch.equal(y16[:7], y7)
    dots = oracle.block_dots_w4a8(W, xq[3]).sum(-1) * 16
    assert np.array_equal(y16[3].cpu().numpy(), dots.astype(np.float32))


def test_tc_arrival_counters_survive_a_smaller_call_before_a_larger_one(k):
    """K-split row tiles count arrivals in the scratch block; a matrix with few tiles followed by one with many once
    found the earlier call's prepared activations where it expected zeroed counters (they now own a fixed region)."""
    import torch

    M, K = 32, 2048
    for N, seed in [(256, 950), (9000, 951), (384, 952), (12800, 953)]:
        W, sc16, _ = synth.int4_weights(N, K, seed=seed)
        x16 = synth.activations_f16(M, K, seed + 30)
        xq, xs = oracle.quantize_int8(x16.astype(np.float32))
        y = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
        k.gemv_w4a8_f16in(y, to_dev(x16.view(np.uint16)), to_dev(W), to_dev(sc16.view(np.uint16)), K, N, M)
        torch.cuda.synchronize()
        assert k.device_status() == 0
        assert max_abs_rel(y.cpu().numpy(), oracle.gemv_w4a8_f64(xq, xs, W, sc16)) < 2e-5, N
