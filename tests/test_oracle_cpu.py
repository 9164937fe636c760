"""The CPU oracle against independent numpy restatements of the same rules and
against the golden outputs of the reference's own CUDA kernels."""
import glob
import os

import numpy as np
import pytest

import oracle
from blackwell_b200 import synth
from tests.util import max_abs_rel

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def np_unpack(packed):
    lo = (packed & 0x0F).astype(np.int32) - 8
    hi = (packed >> 4).astype(np.int32) - 8
    out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), np.int32)
    out[..., 0::2] = lo
    out[..., 1::2] = hi
    return out


def np_round_half_away(x):
    return np.sign(x) * np.floor(np.abs(x) + np.float32(0.5))


def test_quantize_int4_matches_numpy_rule():
    x = synth.activations_f16(3, 512, 1).astype(np.float32)
    x[0, :16] = 0.0  # degenerate block -> scale 1/7
    x[1, 16:32] = 1e-12
    q, sc = oracle.quantize_int4(x)
    xb = x.reshape(3, -1, 16)
    am = np.abs(xb).max(-1)
    sc_ref = np.where(am > np.float32(1e-10), am / np.float32(7), np.float32(1) / np.float32(7)).astype(np.float32)
    assert np.array_equal(sc, sc_ref)
    qi = np.clip(np_round_half_away((xb / sc_ref[..., None]).astype(np.float32)), -8, 7).astype(np.int32)
    assert np.array_equal(np_unpack(q).reshape(3, -1, 16), qi)


def test_quantize_int8_matches_numpy_rule():
    x = synth.activations_f16(2, 1024, 2).astype(np.float32)
    x[0, :16] = 0.0  # degenerate block -> scale 1.0
    q, sc = oracle.quantize_int8(x)
    xb = x.reshape(2, -1, 16)
    am = np.abs(xb).max(-1)
    s = (am / np.float32(127)).astype(np.float32)
    s = np.where(s < np.float32(1e-10), np.float32(1), s)
    assert np.array_equal(sc, s)
    qi = np.clip(np_round_half_away((xb / s[..., None]).astype(np.float32)), -127, 127).astype(np.int8)
    assert np.array_equal(q.reshape(2, -1, 16), qi)


def test_block_dots_and_gemv_flavours_agree():
    N, K, M = 40, 1040, 3  # K = 16 * 65: odd block count
    W, sc16, sc32 = synth.int4_weights(N, K, 3, full_range=True)
    x = synth.activations_f16(M, K, 4).astype(np.float32)
    xq4, xs4 = oracle.quantize_int4(x)
    dots = oracle.block_dots_w4a4(W, xq4[0])
    ref = (np_unpack(W).reshape(N, -1, 16) * np_unpack(xq4[0]).reshape(1, -1, 16)).sum(-1)
    assert np.array_equal(dots, ref)
    y_exact = oracle.gemv_w4a4_exact(xq4, xs4, W, sc32)
    y64 = oracle.gemv_w4a4_f64(xq4, xs4, W, sc32)
    y32, _ = oracle.gemv_w4a4_f32(xq4, xs4, W, sc32, threads=2)
    assert max_abs_rel(y_exact, y64) < 1e-5
    assert max_abs_rel(y32, y64) < 1e-5
    # W4A8
    xq8, xs8 = oracle.quantize_int8(x)
    d8 = oracle.block_dots_w4a8(W, xq8[0])
    ref8 = (np_unpack(W).reshape(N, -1, 16) * xq8[0].astype(np.int32).reshape(1, -1, 16)).sum(-1)
    assert np.array_equal(d8, ref8)
    y8 = oracle.gemv_w4a8_f64(xq8, xs8, W, sc16)
    y8_np = np.empty((M, N), np.float64)
    for m in range(M):
        dm = (np_unpack(W).reshape(N, -1, 16) * xq8[m].astype(np.int32).reshape(1, -1, 16)).sum(-1)
        y8_np[m] = (dm * sc16.astype(np.float64) * xs8[m][None].astype(np.float64)).sum(-1)
    assert np.allclose(y8, y8_np, rtol=1e-12)
    y8f, used = oracle.gemv_w4a8_f32(xq8, xs8, W, sc16, threads=1)
    assert used == 1 and max_abs_rel(y8f, y8) < 1e-5


def test_dequant_row_is_the_format_statement():
    W, _, sc32 = synth.int4_weights(4, 64, 5)
    row = oracle.dequant_row(2, W, sc32)
    ref = np_unpack(W[2]).astype(np.float32) * np.repeat(sc32[2], 16)
    assert np.array_equal(row, ref)


def test_half_conversion_matches_numpy():
    h = np.arange(0, 65536, dtype=np.uint32).astype(np.uint16)
    f = oracle.half_bits_to_float(h)
    ref = h.view(np.float16).astype(np.float32)
    ok = np.isnan(ref) | (f == ref)
    assert ok.all()


def test_rmsnorm_swiglu_argmax_penalty():
    x = synth.activations_f16(2, 4096, 6).astype(np.float32)
    w = synth.norm_weight(4096, 7)
    a = oracle.rmsnorm(x, w)
    b = oracle.rmsnorm(x, w, reforder=True)
    ref = x * w * (1.0 / np.sqrt((x.astype(np.float64) ** 2).mean(-1, keepdims=True) + 1e-6))
    assert np.allclose(a, ref, rtol=1e-6)
    assert np.allclose(b, ref, rtol=1e-5)
    g, u = x[0], x[1]
    assert np.allclose(oracle.swiglu(g, u), g / (1 + np.exp(-g)) * u, rtol=1e-6)
    assert np.allclose(oracle.swiglu_fusedform(g, u), g / (1 + np.exp(-g)) * u, rtol=1e-6)
    assert oracle.argmax(g) == int(np.argmax(g))
    assert oracle.argmax(np.full(10, -2e38, np.float32)) == 0  # nothing beats the -1e38 start value
    pen = oracle.repetition_penalty(g, np.array([3, 5, 3], np.int32), 1.5)
    exp = g.copy()
    for i in (3, 5):
        exp[i] = exp[i] / 1.5 if exp[i] > 0 else exp[i] * 1.5
    assert np.array_equal(pen, exp)
    assert np.array_equal(oracle.repetition_penalty(g, np.array([3], np.int32), 1.0), g)


def test_attention_oracle_against_numpy_softmax():
    nqh, nkv, hd, max_seq, M, pos = 4, 2, 128, 40, 2, 17
    g = synth.rng(8)
    Q = g.normal(size=(M, nqh * hd)).astype(np.float32)
    layer_off = nkv * max_seq * hd
    kv_batch = 2 * layer_off
    Kc = g.normal(size=(M * kv_batch)).astype(np.float32)
    Vc = g.normal(size=(M * kv_batch)).astype(np.float32)
    out = oracle.attention_decode_gqa(Q, Kc, Vc, pos, nqh, nkv, hd, max_seq, M, kv_batch, layer_off)
    for m in range(M):
        for h in range(nqh):
            kvh = h * nkv // nqh
            base = m * kv_batch + layer_off + kvh * max_seq * hd
            K = Kc[base:base + (pos + 1) * hd].reshape(pos + 1, hd).astype(np.float64)
            V = Vc[base:base + (pos + 1) * hd].reshape(pos + 1, hd).astype(np.float64)
            s = K @ Q[m, h * hd:(h + 1) * hd].astype(np.float64) / np.sqrt(hd)
            p = np.exp(s - s.max())
            ref = (p[:, None] * V).sum(0) / (p.sum() + 1e-9)
            assert np.allclose(out[m, h * hd:(h + 1) * hd], ref, rtol=1e-5, atol=1e-6)


def test_head_norm_rope_update_kv():
    nh, hd = 3, 128
    d = synth.rng(9).normal(size=nh * hd).astype(np.float32)
    w = synth.norm_weight(hd, 10)
    hn = oracle.head_norm(d, w, nh, hd).reshape(nh, hd)
    dd = d.reshape(nh, hd).astype(np.float64)
    ref = dd / np.sqrt((dd ** 2).mean(-1, keepdims=True) + 1e-6) * w
    assert np.allclose(hn, ref, rtol=1e-5)
    r = oracle.rope(d, nh, hd, 5).reshape(nh, hd // 2, 2)
    i = np.arange(hd // 2)
    th = 5 * np.power(1e6, -2.0 * i / hd)
    x, y = dd.reshape(nh, hd // 2, 2)[..., 0], dd.reshape(nh, hd // 2, 2)[..., 1]
    assert np.allclose(r[..., 0], x * np.cos(th) - y * np.sin(th), atol=1e-4)
    assert np.allclose(r[..., 1], x * np.sin(th) + y * np.cos(th), atol=1e-4)
    kc = np.zeros((nh, 8, hd), np.float32)
    vc = np.zeros((nh, 8, hd), np.float32)
    oracle.update_kv(kc, vc, d, -d, 3, nh, hd, 8)
    assert np.array_equal(kc[:, 3], d.reshape(nh, hd)) and np.array_equal(vc[:, 3], -d.reshape(nh, hd))
    assert not kc[:, :3].any() and not kc[:, 4:].any()


# ------------------------------------------------------------------ golden pins
def _golden_files():
    return sorted(glob.glob(os.path.join(GOLDEN, "ref_*.npz")))


@pytest.mark.parametrize("path", _golden_files() or [None])
def test_oracle_matches_reference_cuda_goldens(path):
    """Outputs of the reference's own CUDA kernels (rebuilt for sm_100a, run on a
    B200 by tests/golden/make_golden.py) on seeded inputs; the oracle must
    reproduce the integer outputs bit for bit and the exact-order GEMV bit for bit."""
    if path is None:
        pytest.skip("no reference fixtures committed yet")
    from tests.golden import make_golden as mg

    z = np.load(path)
    case = mg.CASES[str(z["case"])]
    inp = mg.make_inputs(case)
    q4, s4 = oracle.quantize_int4(inp["x32"])
    assert np.array_equal(q4, z["q4"]) and np.array_equal(s4, z["s4"])
    q8, s8 = oracle.quantize_int8(inp["x32"])
    assert np.array_equal(q8, z["q8"]) and np.array_equal(s8.reshape(-1), z["s8"].reshape(-1))
    y = oracle.gemv_w4a4_exact(q4, s4, inp["W"], inp["sc32"])
    assert np.array_equal(y, z["y_w4a4"]), f"exact-order oracle differs: {max_abs_rel(y, z['y_w4a4'])}"
    y64 = oracle.gemv_w4a4_f64(q4, s4, inp["W"], inp["sc32"])
    assert max_abs_rel(z["y_w4a4"], y64) < 1e-5
    if "rms" in z:
        ref = oracle.rmsnorm(inp["x32"], inp["nw"], reforder=True)
        assert np.allclose(z["rms"], ref, rtol=3e-6, atol=1e-7)
    if "swiglu" in z:
        assert np.allclose(z["swiglu"], oracle.swiglu(inp["x32"][0], inp["x32"][-1]), rtol=2e-6, atol=1e-7)
    if "attn" in z:
        a = mg.attn_inputs(case)
        ref = oracle.attention_decode_gqa(a["Q"], a["Kc"], a["Vc"], a["pos"], a["nqh"], a["nkv"], 128, a["max_seq"],
                                          a["M"], a["kv_batch"], a["layer_off"])
        assert max_abs_rel(z["attn"], ref) < 1e-4
    if "argmax" in z:
        assert int(z["argmax"]) == oracle.argmax(y[0])
