"""One synthetic decode step of a small Qwen3-shaped model through the C ABI against the same chain of oracle
routines on the CPU (the reference's per-layer sequence, server/inference_server_int4_batched.cu:253-298, with
int8 activations and a binary16 cache).  Also the glue kernels on their own."""
import numpy as np
import pytest

import oracle
from blackwell_b200 import synth
from blackwell_b200.shapes import ModelShape
from tests.util import max_abs_rel, to_dev

pytestmark = pytest.mark.gpu

SMALL = ModelShape("small", layers=2, hidden=256, inter=416, n_q_heads=4, n_kv_heads=2, head_dim=128, vocab=1003)
# four query heads per kv head: the fused attention form with quantized output, and at batch 1 the norm-pending hand-over
SMALL_GQ4 = ModelShape("small-gq4", layers=2, hidden=256, inter=416, n_q_heads=8, n_kv_heads=2, head_dim=128, vocab=1003)


class HostWeights:
    def __init__(self):
        self.np = {}

    def __call__(self, N, K, sd):
        if N == "embed":
            V, H = K, sd
            e = synth.activations_f16(V, H, 4242)
            self.np["embed"] = e
            return to_dev(e.view(np.uint16)).view(__import__("torch").float16)
        W, sc16, _ = synth.int4_weights(N, K, sd)
        self.np[sd] = (W, sc16)
        return to_dev(W), to_dev(sc16.view(np.uint16)).view(__import__("torch").float16)


def cpu_gemv(x, W, sc16):
    q, s = oracle.quantize_int8(np.ascontiguousarray(x, np.float32))
    return oracle.gemv_w4a8_f64(q, s, W, sc16).astype(np.float32)


@pytest.mark.parametrize("M,s", [(3, SMALL), (16, SMALL), (1, SMALL_GQ4), (3, SMALL_GQ4), (8, SMALL_GQ4)])
def test_decode_step_matches_cpu_chain(cuda, M, s):
    """Batch 3 runs the dp4a GEMV kernel, batch 8 and 16 the mma.sync one; with four query heads per kv head the fused
    attention form, and at batch 1 the norm-pending hand-over between the GEMVs."""
    import torch

    from blackwell_b200.decode import ROPE_BASE, DecodeEngine

    max_seq, ctx = 96, 40
    hw = HostWeights()
    eng = DecodeEngine(s, M, max_seq, cuda, seed=5, host_weights=hw)
    eng.fill_cache(ctx)
    pos0 = np.array(([ctx - 1, ctx - 5, 3] + [(5 * i) % ctx for i in range(M - 3)])[:M], np.int32)
    eng.pos.copy_(torch.from_numpy(pos0))
    toks = np.array(([7, 1002, 500] + [(91 * i + 13) % s.vocab for i in range(M - 3)])[:M], np.int32)
    eng.set_tokens(toks)
    Kc = eng.kc.cpu().numpy().copy()
    Vc = eng.vc.cpu().numpy().copy()
    eng.step()
    torch.cuda.synchronize()

    # ---- CPU chain
    nq, nkv, H, I = s.n_q_heads, s.n_kv_heads, s.hidden, s.inter
    x = hw.np["embed"][toks].astype(np.float32)
    Kc = Kc.reshape(M, s.layers, nkv, max_seq, 128)
    Vc = Vc.reshape(M, s.layers, nkv, max_seq, 128)
    for l, L in enumerate(eng.layers):
        sd = 5 + 1000 * l
        qkv = cpu_gemv(oracle.rmsnorm(x, L["rn_in"].cpu().numpy()), *hw.np[sd + 1])
        q = np.empty((M, nq * 128), np.float32)
        for m in range(M):
            qm = oracle.rope(oracle.head_norm(qkv[m, :nq * 128], L["qn"].cpu().numpy(), nq, 128), nq, 128, int(pos0[m]))
            km = oracle.rope(oracle.head_norm(qkv[m, nq * 128:(nq + nkv) * 128], L["kn"].cpu().numpy(), nkv, 128),
                             nkv, 128, int(pos0[m]))
            q[m] = qm
            Kc[m, l, :, pos0[m]] = km.reshape(nkv, 128).astype(np.float16)
            Vc[m, l, :, pos0[m]] = qkv[m, (nq + nkv) * 128:].reshape(nkv, 128).astype(np.float16)
        attn = oracle.attention_decode_f16kv(q, np.ascontiguousarray(Kc[:, l]), np.ascontiguousarray(Vc[:, l]), pos0,
                                             nq, nkv, 128, max_seq, M)
        x = x + cpu_gemv(attn, *hw.np[sd + 2])
        gu = cpu_gemv(oracle.rmsnorm(x, L["rn_post"].cpu().numpy()), *hw.np[sd + 3])
        act = oracle.swiglu(np.ascontiguousarray(gu[:, :I]), np.ascontiguousarray(gu[:, I:]))
        x = x + cpu_gemv(act, *hw.np[sd + 4])
    logits = cpu_gemv(oracle.rmsnorm(x, eng.rn_final.cpu().numpy()), *hw.np[5 + 900001])

    # A rounding tie of the int8 activation quantizer resolved the other way (rsqrtf, summation order) moves one
    # element by a whole step and with it one sequence's later values by up to a percent of the largest one; every
    # other sequence agrees to fp32 rounding.  So: all sequences inside the loose bound, all but a few inside the tight.
    def per_seq(a, b):
        return np.abs(a.astype(np.float64) - b).max(axis=1) / np.abs(b).max()

    ex, el = per_seq(eng.x.cpu().numpy(), x), per_seq(eng.logits.cpu().numpy(), logits)
    print("per-sequence max abs rel: x", np.array2string(ex, precision=2), "logits", np.array2string(el, precision=2))
    tol = 2e-2
    assert ex.max() < tol and el.max() < tol, (ex, el)
    assert (el > 1e-4).sum() <= max(1, M // 4), el
    got_k = eng.kc.cpu().numpy().reshape(M, s.layers, nkv, max_seq, 128).astype(np.float32)
    assert max_abs_rel(got_k, Kc.astype(np.float32)) < 5e-3
    # greedy ids: equal wherever the CPU's top-2 margin exceeds the numerical noise
    ids = eng.tokens.cpu().numpy()
    for m in range(M):
        top = np.sort(logits[m])[-2:]
        if top[1] - top[0] > (2.5 * el[m] + 1e-4) * np.abs(logits).max():
            assert ids[m] == int(np.argmax(logits[m]))
    assert np.array_equal(eng.pos.cpu().numpy(), pos0 + 1)


def test_decode_step_graph_replay_is_deterministic(cuda):
    import torch

    from blackwell_b200.decode import DecodeEngine

    eng = DecodeEngine(SMALL, 2, 64, cuda, seed=9)
    eng.fill_cache(20)
    eng.set_tokens([5, 6])
    eng.step()  # warm-up outside capture (first-use allocations)
    torch.cuda.synchronize()

    def run():
        eng.pos.fill_(19)
        eng.set_tokens([5, 6])
        g.replay()
        g.replay()
        torch.cuda.synchronize()
        return eng.tokens.cpu().numpy().copy(), eng.logits.cpu().numpy().copy()

    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        eng.step()
    t1, l1 = run()
    t2, l2 = run()
    assert np.array_equal(t1, t2) and np.array_equal(l1, l2)
    assert np.array_equal(eng.pos.cpu().numpy(), [21, 21])


def test_qk_norm_rope_kv_and_embed_and_batched_argmax(cuda):
    import torch

    from blackwell_b200 import kernels as k

    M, nq, nkv, max_seq = 3, 8, 2, 50
    g = synth.rng(400)
    qkv = g.normal(size=(M, (nq + 2 * nkv) * 128)).astype(np.float32)
    qn, kn = synth.norm_weight(128, 401), synth.norm_weight(128, 402)
    pos = np.array([0, 17, 49], np.int32)
    layers, layer = 2, 1
    kv_layer = nkv * max_seq * 128
    kc = torch.zeros((M, layers * kv_layer), dtype=torch.float16, device="cuda")
    vc = torch.zeros_like(kc)
    q = torch.empty((M, nq * 128), dtype=torch.float32, device="cuda")
    k.qk_norm_rope_kv_f16(q, kc, vc, to_dev(qkv), to_dev(qn), to_dev(kn), to_dev(pos), nq, nkv, 128, max_seq, M,
                          layers * kv_layer, layer * kv_layer, 1e-6, 1e6)
    kc_n = kc.cpu().numpy().reshape(M, layers, nkv, max_seq, 128)
    vc_n = vc.cpu().numpy().reshape(M, layers, nkv, max_seq, 128)
    for m in range(M):
        qr = oracle.rope(oracle.head_norm(qkv[m, :nq * 128], qn, nq, 128), nq, 128, int(pos[m]))
        kr = oracle.rope(oracle.head_norm(qkv[m, nq * 128:(nq + nkv) * 128], kn, nkv, 128), nkv, 128, int(pos[m]))
        assert np.allclose(q[m].cpu().numpy(), qr, rtol=1e-4, atol=2e-4)
        assert np.allclose(kc_n[m, layer, :, pos[m]].astype(np.float32).reshape(-1), kr, rtol=2e-3, atol=2e-3)
        assert np.array_equal(vc_n[m, layer, :, pos[m]].reshape(-1), qkv[m, (nq + nkv) * 128:].astype(np.float16))
    assert not kc_n[:, 0].any() and kc_n[0, layer, :, 1:].sum() == 0  # nothing else was touched

    V, H = 300, 256
    table = synth.activations_f16(V, H, 403)
    toks = np.array([0, 299, 123], np.int32)
    x = torch.empty((M, H), dtype=torch.float32, device="cuda")
    k.embed_gather_f16(x, to_dev(table.view(np.uint16)), to_dev(toks), H, V, M)
    assert np.array_equal(x.cpu().numpy(), table[toks].astype(np.float32))

    Vv = 151643
    logits = synth.rng(404).normal(size=(M, Vv)).astype(np.float32)
    logits[1, 77] = logits[1].max()  # tie -> lowest index
    ids = torch.zeros(M, dtype=torch.int32, device="cuda")
    p = to_dev(pos)
    for _ in range(2):  # twice: the tickets are reset by the kernel
        k.sample_argmax_batched(to_dev(logits), Vv, Vv, M, ids, p)
    assert [int(i) for i in ids.cpu()] == [oracle.argmax(logits[m]) for m in range(M)]
    assert np.array_equal(p.cpu().numpy(), pos + 2)


@pytest.mark.parametrize("nq,nkv", [(8, 2), (8, 1), (32, 8)])
def test_fused_norm_rope_kv_attention_equals_the_two_launches(cuda, nq, nkv):
    """bw_attention_decode_f16kv_fused against bw_qk_norm_rope_kv_f16 + bw_attention_decode_f16kv on the same inputs:
    same arithmetic, so the attention output and the cache rows must be bit-identical; positions at 0, inside and at
    the end of a split, beyond the context hint, and one outside the cache (not written)."""
    import torch

    from blackwell_b200 import kernels as k

    M, max_seq, hint = 6, 1400, 800   # three splits of 268 positions
    g = synth.rng(440 + nq + nkv)
    qkv = to_dev(g.normal(size=(M, (nq + 2 * nkv) * 128)).astype(np.float32))
    qn, kn = to_dev(synth.norm_weight(128, 441)), to_dev(synth.norm_weight(128, 442))
    pos = to_dev(np.array([0, 267, 268, 799, 1300, 1400], np.int32))
    layers, layer = 2, 1
    kv_layer = nkv * max_seq * 128
    base = synth.kv_cache_f16((M, layers * kv_layer), 443)
    kc1 = to_dev(base.view(np.uint16)).view(torch.float16)
    vc1 = to_dev(synth.kv_cache_f16((M, layers * kv_layer), 444).view(np.uint16)).view(torch.float16)
    kc2, vc2 = kc1.clone(), vc1.clone()
    q = torch.empty((M, nq * 128), dtype=torch.float32, device="cuda")
    out1 = torch.empty((M, nq * 128), dtype=torch.float32, device="cuda")
    out2 = torch.full_like(out1, float("nan"))
    k.qk_norm_rope_kv_f16(q, kc1, vc1, qkv, qn, kn, pos, nq, nkv, 128, max_seq, M, layers * kv_layer, layer * kv_layer,
                          1e-6, 1e6)
    k.attention_decode_f16kv(out1, q, kc1, vc1, pos, hint, nq, nkv, 128, max_seq, M, layers * kv_layer, layer * kv_layer)
    k.attention_decode_f16kv_fused(out2, qkv, qn, kn, kc2, vc2, pos, hint, nq, nkv, 128, max_seq, M, layers * kv_layer,
                                   layer * kv_layer, 1e-6, 1e6)
    torch.cuda.synchronize()
    assert torch.equal(kc1, kc2) and torch.equal(vc1, vc2)
    assert torch.equal(out1, out2)
    # the quantized second output: the bits of bw_quantize_int8 applied to the float result, with split merge (hint
    # 800 of up to 1400 positions) and without (a hint of 8 positions gives one open-ended split)
    for h in (hint, 8):
        kc3, vc3 = kc1.clone(), vc1.clone()
        out3 = torch.full_like(out1, float("nan"))
        oq = torch.zeros((M, nq * 128), dtype=torch.int8, device="cuda")
        os_ = torch.zeros((M, nq * 8), dtype=torch.float32, device="cuda")
        k.attention_decode_f16kv_fused_q8(out3, oq, os_, qkv, qn, kn, kc3, vc3, pos, h, nq, nkv,
                                          128, max_seq, M, layers * kv_layer, layer * kv_layer, 1e-6, 1e6)
        torch.cuda.synchronize()
        ref_q, ref_s = oracle.quantize_int8(out3.cpu().numpy())
        assert np.array_equal(oq.cpu().numpy(), ref_q) and np.array_equal(os_.cpu().numpy(), ref_s)
        if h == hint:
            assert torch.equal(out3, out2)
        # the O projection on the quantized operand equals the one that quantizes the float result itself
        W, sc16, _ = synth.int4_weights(256, nq * 128, seed=445)
        Wd, sd = to_dev(W), to_dev(sc16.view(np.uint16))
        res = to_dev(synth.activations_f16(M, 256, 446).astype(np.float32))
        y1, y2 = res.clone(), res.clone()
        k.gemv_w4a8_decode(y1, 0, y1, out3, None, 0, None, 0.0, Wd, sd, nq * 128, 256, M)
        k.gemv_w4a8_q8_decode(y2, 0, y2, oq, os_, Wd, sd, nq * 128, 256, M)
        assert torch.equal(y1, y2)
    assert k.device_status() == 0


def test_tensor_parallel_argmax_candidates_and_merge(cuda):
    """The vocabulary cut into three ranks' slices: per-slice candidates + merge give the ids of the full argmax
    (ties to the lowest global index) and advance the positions once."""
    import torch

    from blackwell_b200 import kernels as k

    M, V, world = 5, 10007, 3
    logits = synth.rng(430).normal(size=(M, V)).astype(np.float32)
    logits[1, 9000] = logits[1, 17] = logits[1].max() + 1.0      # a tie across two slices -> index 17
    logits[2, :] = -np.inf                                       # nothing qualifies -> index 0
    bounds = [0, 3336, 6672, V]
    cand_all = torch.zeros((world, M, 2), dtype=torch.int32, device="cuda")
    for r in range(world):
        sl = to_dev(np.ascontiguousarray(logits[:, bounds[r]:bounds[r + 1]]))
        n = bounds[r + 1] - bounds[r]
        k.sample_argmax_candidates(sl, n, n, M, bounds[r], cand_all[r])
    ids = torch.zeros(M, dtype=torch.int32, device="cuda")
    pos = to_dev(np.array([0, 1, 2, 3, 9], np.int32))
    k.sample_argmax_merge(cand_all, world, M, ids, pos, 9)
    assert [int(i) for i in ids.cpu()] == [oracle.argmax(logits[m]) for m in range(M)]
    assert pos.cpu().tolist() == [1, 2, 3, 4, 9]
    vals = cand_all.cpu().numpy()[..., 0].view(np.float32)
    assert vals[0, 1] == logits[1, 17] and vals[2, 1] == logits[1, 9000]


def test_positions_outside_the_cache_are_never_written(cuda):
    """A sequence whose position has reached max_seq (a replayed step that ran past the cache) must leave the cache
    and everything behind it alone, and the batched argmax must stop advancing positions at its limit."""
    import torch

    from blackwell_b200 import kernels as k

    M, nq, nkv, max_seq = 3, 4, 2, 16
    g = synth.rng(420)
    qkv = g.normal(size=(M, (nq + 2 * nkv) * 128)).astype(np.float32)
    qn, kn = synth.norm_weight(128, 421), synth.norm_weight(128, 422)
    kv_layer = nkv * max_seq * 128
    canary = 4096
    # one allocation: [K cache][canary]; the last sequence's last head ends where the canary begins
    buf_k = torch.full((M * kv_layer + canary,), 7.0, dtype=torch.float16, device="cuda")
    buf_v = torch.full((M * kv_layer + canary,), 7.0, dtype=torch.float16, device="cuda")
    q = torch.empty((M, nq * 128), dtype=torch.float32, device="cuda")
    pos = np.array([3, max_seq, max_seq + 5], np.int32)
    k.qk_norm_rope_kv_f16(q, buf_k, buf_v, to_dev(qkv), to_dev(qn), to_dev(kn), to_dev(pos), nq, nkv, 128, max_seq, M,
                          kv_layer, 0, 1e-6, 1e6)
    torch.cuda.synchronize()
    for buf in (buf_k, buf_v):
        h = buf.cpu().numpy()
        cache = h[:M * kv_layer].reshape(M, nkv, max_seq, 128)
        assert (h[M * kv_layer:] == 7.0).all()                 # nothing behind the cache
        assert (cache[1:] == 7.0).all()                        # the two out-of-range sequences wrote nothing
        assert (cache[0, :, 3] != 7.0).any() and (np.delete(cache[0], 3, axis=1) == 7.0).all()
    # the fp32 reference-format update with a device position outside the cache
    kc = torch.full((nkv * max_seq * 128 + canary,), 7.0, dtype=torch.float32, device="cuda")
    vc = kc.clone()
    new = to_dev(g.normal(size=nkv * 128).astype(np.float32))
    k.update_kv_cache_device(kc, vc, new, new, 0, to_dev(np.array([max_seq], np.int32)), nkv, 128, max_seq)
    torch.cuda.synchronize()
    assert (kc == 7.0).all() and (vc == 7.0).all()
    # positions stop at the limit
    logits = to_dev(g.normal(size=(M, 1000)).astype(np.float32))
    ids = torch.zeros(M, dtype=torch.int32, device="cuda")
    p = to_dev(np.array([3, max_seq - 2, max_seq - 1], np.int32))
    for _ in range(3):
        k.sample_argmax_batched(logits, 1000, 1000, M, ids, p, max_seq - 1)
    assert p.cpu().tolist() == [6, max_seq - 1, max_seq - 1]


def test_gemv_decode_entry_residual_and_strides(cuda):
    import torch

    from blackwell_b200 import kernels as k

    M, K, N = 3, 416, 200
    W, sc16, _ = synth.int4_weights(N, K, 410)
    gu = synth.activations_f16(M, 2 * K, 411).astype(np.float32)
    res = synth.activations_f16(M, N + 8, 412).astype(np.float32)
    y = to_dev(res.copy())
    gud = to_dev(gu)
    k.gemv_w4a8_decode(y, N + 8, y, gud, gud[:, K:], 2 * K, None, 0.0, to_dev(W), to_dev(sc16.view(np.uint16)), K, N,
                       M)
    act = oracle.swiglu(np.ascontiguousarray(gu[:, :K]), np.ascontiguousarray(gu[:, K:]))
    ref = res[:, :N] + cpu_gemv(act, W, sc16)
    out = y.cpu().numpy()
    assert max_abs_rel(out[:, :N], ref) < 1e-3
    assert np.array_equal(out[:, N:], res[:, N:])  # the padding columns are untouched


@pytest.mark.parametrize("M,from_swiglu,K1", [(1, False, 1024), (1, True, 1024), (1, True, 12288), (8, False, 1024),
                                              (8, True, 12288), (5, True, 2048)])
def test_norm_pending_hand_over_between_two_gemvs(cuda, M, from_swiglu, K1):
    """bw_gemv_w4a8_pending at one sequence (dp4a kernel) and at 5..8 (mma.sync kernel): the producer
    (y = residual + W1 x) also emits q8(y * w_norm) block by block and the blocks' sums of y^2; the consumer applies
    1/rms to the block scales.  The emitted integers and scales are those of the quantize rule on y * w_norm (bit for
    bit), and the consumer's output is W2 . q8(rmsnorm(y, w_norm)) within the tolerance of the fused-norm prologue (one
    float rounding more).  K1 = 12288 at one sequence: the producer's tiles hold 8 rows, half a block of the consumer."""
    import torch

    from blackwell_b200 import kernels as k

    H, N2, eps = 512, 300, 1e-6
    W1, s1, _ = synth.int4_weights(H, K1, 470)
    W2, s2, _ = synth.int4_weights(N2, H, 471)
    res = synth.activations_f16(M, H, 472).astype(np.float32)
    nw = synth.norm_weight(H, 473)
    W1d, s1d, W2d, s2d = to_dev(W1), to_dev(s1.view(np.uint16)), to_dev(W2), to_dev(s2.view(np.uint16))
    y = to_dev(res.copy())
    nq = torch.zeros((M, H), dtype=torch.int8, device="cuda")
    ns = torch.zeros((M, H // 16), dtype=torch.float32, device="cuda")
    nss = torch.zeros((M, H // 16), dtype=torch.float32, device="cuda")
    if from_swiglu:
        gu = synth.activations_f16(M, 2 * K1, 474).astype(np.float32)
        gud = to_dev(gu)
        k.gemv_w4a8_pending(y, y, W1d, s1d, K1, H, gate=gud, up=gud[:, K1:].data_ptr(), next_norm_w=to_dev(nw), next_q=nq,
                            next_scale=ns, next_block_sumsq=nss, M=M, x_stride=2 * K1)
        x1 = oracle.swiglu(np.ascontiguousarray(gu[:, :K1]), np.ascontiguousarray(gu[:, K1:]))
    else:
        x1 = synth.activations_f16(M, K1, 475).astype(np.float32)
        xq, xs = oracle.quantize_int8(x1)
        k.gemv_w4a8_pending(y, y, W1d, s1d, K1, H, x_q=to_dev(xq), x_scale=to_dev(xs), next_norm_w=to_dev(nw), next_q=nq,
                            next_scale=ns, next_block_sumsq=nss, M=M)
    torch.cuda.synchronize()
    yh = y.cpu().numpy()
    assert max_abs_rel(yh, res + cpu_gemv(x1, W1, s1)) < 1e-3
    # what the producer emitted, against the rule applied to the y it wrote
    ref_q, ref_s = oracle.quantize_int8((yh * nw).astype(np.float32))
    assert np.array_equal(nq.cpu().numpy(), ref_q) and np.array_equal(ns.cpu().numpy(), ref_s)
    ss = (yh.astype(np.float64) ** 2).reshape(M, -1, 16).sum(2)
    assert np.allclose(nss.cpu().numpy(), ss, rtol=1e-5)
    # the consumer
    out = torch.full((M, N2), float("nan"), dtype=torch.float32, device="cuda")
    k.gemv_w4a8_pending(out, None, W2d, s2d, H, N2, x_q=nq, x_scale=ns, x_block_sumsq=nss, eps=eps, M=M)
    ref = cpu_gemv(oracle.rmsnorm(yh, nw), W2, s2)
    assert max_abs_rel(out.cpu().numpy(), ref) < 1e-3
    # and against this library's fused-norm prologue on the same y
    out2 = torch.empty_like(out)
    k.gemv_w4a8_decode(out2, 0, None, y, None, 0, to_dev(nw), eps, W2d, s2d, H, N2, M)
    assert max_abs_rel(out.cpu().numpy(), out2.cpu().numpy()) < 1e-3
    assert k.device_status() == 0
