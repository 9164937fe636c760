"""The C decode-step driver (bw_decode_*: csrc/decode_engine.cu) on a small synthetic weight tree, against the same
chain of oracle routines on the CPU (the reference's per-layer sequence, server/inference_server_int4_batched.cu:
253-298): sequences with prompts of different lengths advance together, one captured-graph replay per token, in
both activation formats (8: int8 activations / binary16 weight scales; 4: the reference's own INT4 arithmetic)."""
import numpy as np
import pytest

import oracle
from blackwell_b200 import synth
from blackwell_b200.shapes import ModelShape
from tests.util import max_abs_rel

pytestmark = pytest.mark.gpu

SMALL = ModelShape("small-tree", layers=2, hidden=256, inter=416, n_q_heads=4, n_kv_heads=2, head_dim=128, vocab=1003)
# four query heads per kv head: the fused attention form, and with it the norm-pending hand-over at batch 1
SMALL_GQ4 = ModelShape("small-tree-gq4", layers=2, hidden=256, inter=416, n_q_heads=8, n_kv_heads=2, head_dim=128,
                       vocab=1003)
ROPE_BASE = 1000000.0


class CpuModel:
    """The tree's weights on the host and the oracle chain of one decode step with a binary16 cache."""

    def __init__(self, root, shape, act_bits, batch, max_seq):
        from blackwell_b200 import weight_files as wf

        self.s, self.act_bits = shape, act_bits
        rd = lambda name: wf.read_w4(f"{root}/{name}")
        self.layers = []
        qk = wf.read_f32(f"{root}/qk_norms.f32", shape.layers * 256).reshape(shape.layers, 2, 128)
        for l in range(shape.layers):
            q, k, v = rd(f"{l}_self_attn.q_proj"), rd(f"{l}_self_attn.k_proj"), rd(f"{l}_self_attn.v_proj")
            g, u = rd(f"{l}_mlp.gate_proj"), rd(f"{l}_mlp.up_proj")
            self.layers.append({
                "qkv": (np.concatenate([q[0], k[0], v[0]]), np.concatenate([q[1], k[1], v[1]])),
                "o": rd(f"{l}_self_attn.o_proj"), "gu": (np.concatenate([g[0], u[0]]), np.concatenate([g[1], u[1]])),
                "down": rd(f"{l}_mlp.down_proj"),
                "rn_in": wf.read_f32(f"{root}/{l}_input_layernorm.f32", shape.hidden),
                "rn_post": wf.read_f32(f"{root}/{l}_post_attention_layernorm.f32", shape.hidden),
                "qn": qk[l, 0], "kn": qk[l, 1]})
        self.lm = rd("lm_head")
        self.rn_final = wf.read_f32(f"{root}/final_norm.f32", shape.hidden)
        ew, es = rd("embed_tokens")
        nib = np.stack([ew & 0x0F, ew >> 4], axis=-1).reshape(ew.shape[0], -1).astype(np.float32) - 8.0
        self.embed = (nib * np.repeat(es, 16, axis=1)).astype(np.float32)   # (nibble - 8) * scale, as the reference
        self.Kc = np.zeros((batch, shape.layers, shape.n_kv_heads, max_seq, 128), np.float16)
        self.Vc = np.zeros_like(self.Kc)
        self.max_seq = max_seq

    def gemv(self, x, W):
        packed, sc32 = W
        x = np.ascontiguousarray(x, np.float32)
        if self.act_bits == 4:
            q, s = oracle.quantize_int4(x)
            return oracle.gemv_w4a4_f64(q, s, packed, sc32).astype(np.float32)
        q, s = oracle.quantize_int8(x)
        return oracle.gemv_w4a8_f64(q, s, packed, sc32.astype(np.float16)).astype(np.float32)

    def step(self, tokens, pos):
        s = self.s
        M, nq, nkv, I = len(tokens), s.n_q_heads, s.n_kv_heads, s.inter
        x = self.embed[np.asarray(tokens)]
        for l, L in enumerate(self.layers):
            qkv = self.gemv(oracle.rmsnorm(x, L["rn_in"]), L["qkv"])
            q = np.empty((M, nq * 128), np.float32)
            for m in range(M):
                q[m] = oracle.rope(oracle.head_norm(qkv[m, :nq * 128], L["qn"], nq, 128), nq, 128, int(pos[m]))
                km = oracle.rope(oracle.head_norm(qkv[m, nq * 128:(nq + nkv) * 128], L["kn"], nkv, 128), nkv, 128, int(pos[m]))
                self.Kc[m, l, :, pos[m]] = km.reshape(nkv, 128).astype(np.float16)
                self.Vc[m, l, :, pos[m]] = qkv[m, (nq + nkv) * 128:].reshape(nkv, 128).astype(np.float16)
            attn = oracle.attention_decode_f16kv(q, np.ascontiguousarray(self.Kc[:, l]), np.ascontiguousarray(self.Vc[:, l]),
                                                 np.asarray(pos, np.int32), nq, nkv, 128, self.max_seq, M)
            x = x + self.gemv(attn, L["o"])
            gu = self.gemv(oracle.rmsnorm(x, L["rn_post"]), L["gu"])
            act = oracle.swiglu(np.ascontiguousarray(gu[:, :I]), np.ascontiguousarray(gu[:, I:]))
            x = x + self.gemv(act, L["down"])
        logits = self.gemv(oracle.rmsnorm(x, self.rn_final), (self.lm[0][:s.vocab], self.lm[1][:s.vocab]))
        return x, logits


@pytest.mark.parametrize("act_bits,use_graph,M,s", [(8, True, 3, SMALL), (4, True, 3, SMALL), (8, False, 3, SMALL),
                                                    (8, True, 1, SMALL_GQ4), (8, True, 3, SMALL_GQ4)])
def test_driver_generation_matches_cpu_chain(cuda, tmp_path, act_bits, use_graph, M, s):
    """Batch 3: prep launches before the GEMVs; batch 1 with four query heads per kv head (int8): the fused attention
    with quantized output and the norm-pending hand-over between the GEMVs."""
    import torch

    from blackwell_b200 import kernels as k
    from blackwell_b200 import weight_files as wf
    from blackwell_b200.decode_driver import DecodeDriver

    max_seq, max_new = 32, 4
    root = str(tmp_path / "tree")
    wf.write_synthetic_tree(root, s, seed=7)
    drv = DecodeDriver(s, root, batch=M, max_seq=max_seq, max_prompt=8, max_new=max_new, act_bits=act_bits,
                       use_graph=use_graph)
    cpu = CpuModel(root, s, act_bits, M, max_seq)
    prompts = [[5, 900, 17], [1002], [44, 45, 46, 47, 48]][:M]
    lens = [len(p) for p in prompts]
    try:
        for rep in range(2):   # a second generation on the same engine starts from clean positions
            drv.begin(prompts)
            buf = drv.buffers()
            last = [0] * M          # ids sampled by the previous step (CPU side)
            gen_cpu = [[] for _ in range(M)]
            trusted = [True] * M    # a sequence stays comparable until a near-tie of its logits
            steps = max(lens) + max_new - 1
            tol = 5e-3 if act_bits == 4 else 2e-3   # int4 rounding ties flip whole quantization steps
            # Rounding ties: the attention result (binary16 cache, tensor-core products) differs from the CPU chain's by
            # ~1e-5, and the norm-pending hand-over (batch 1) rounds y * w * 127 / amax where the chain rounds
            # (y * rstd * w) / (amax / 127); where that moves an activation across a tie of the int8 quantize, that step's
            # logits move by a quantization step of one input -- visible on this model of 256 hidden values, more often
            # with 1024 attention outputs per sequence than with 512.  Steps are independent here (the CPU side restarts
            # from the device's caches), so: every step inside a loose bound, all but a few inside the tight one.
            loose_steps = 0
            for st in range(steps):
                pos = [st] * M
                toks = [prompts[m][st] if st < lens[m] else last[m] for m in range(M)]
                drv.step()
                torch.cuda.synchronize()
                _, logits = cpu.step(toks, pos)
                loose_any = False   # a tie flip in this step: its later layers' cache rows moved too
                got = buf["logits"].cpu().numpy()
                ids = buf["sampled"].cpu().numpy()
                for m in range(M):
                    if not trusted[m]:
                        continue
                    err = max_abs_rel(got[m], logits[m])
                    loose_now = tol <= err < 2e-2
                    loose_steps += int(loose_now)
                    loose_any = loose_any or loose_now
                    assert err < tol or loose_now, (rep, st, m)
                    top = np.sort(logits[m])[-2:]
                    clear = top[1] - top[0] > 4 * max(tol, 2 * err) * np.abs(logits[m]).max()
                    if clear:
                        assert ids[m] == int(np.argmax(logits[m])), (rep, st, m)
                    else:
                        trusted[m] = ids[m] == int(np.argmax(logits[m]))
                    last[m] = int(ids[m])            # follow the device's choice so the caches stay aligned
                    if st + 1 >= lens[m] and len(gen_cpu[m]) < max_new:
                        gen_cpu[m].append(int(ids[m]))
                # the rows this step wrote into the caches; then the CPU side continues from the device's caches, so
                # that every step is compared on its own and rounding differences of earlier steps do not pile up
                kc, vc = buf["kc"].cpu().numpy(), buf["vc"].cpu().numpy()
                assert loose_steps <= 3, (rep, st, loose_steps)
                if all(trusted) and not loose_any:
                    assert max_abs_rel(kc[:, :, :, st].astype(np.float32), cpu.Kc[:, :, :, st].astype(np.float32)) < tol
                    assert max_abs_rel(vc[:, :, :, st].astype(np.float32), cpu.Vc[:, :, :, st].astype(np.float32)) < tol
                cpu.Kc[:], cpu.Vc[:] = kc, vc
                assert np.array_equal(buf["pos"].cpu().numpy(), np.full(M, st + 1))
            gen = drv.result()
            for m in range(M):
                if trusted[m]:
                    assert gen[m, :len(gen_cpu[m])].tolist() == gen_cpu[m], (rep, m, gen[m], gen_cpu[m])
                    assert (gen[m, len(gen_cpu[m]):] == -1).all()
            assert any(trusted)
            cpu.Kc[:] = 0
            cpu.Vc[:] = 0
        assert k.device_status() == 0
    finally:
        drv.close()


def test_driver_rejects_bad_configurations(cuda, tmp_path):
    from blackwell_b200 import weight_files as wf
    from blackwell_b200.decode_driver import DecodeDriver
    from blackwell_b200.kernels import KernelError

    root = str(tmp_path / "tree")
    wf.write_synthetic_tree(root, SMALL, seed=8)
    with pytest.raises(KernelError):     # no such directory
        DecodeDriver(SMALL, str(tmp_path / "nothing"), 2, 16, 4, 4)
    wrong = ModelShape("wrong", 2, 512, 416, 4, 2, 128, 1003)
    with pytest.raises(KernelError):     # shape does not match the files
        DecodeDriver(wrong, root, 2, 16, 4, 4)
    with pytest.raises(KernelError):     # unsupported activation format
        DecodeDriver(SMALL, root, 2, 16, 4, 4, act_bits=6)
    drv = DecodeDriver(SMALL, root, 2, 16, 4, 4)
    try:
        with pytest.raises(KernelError):  # a prompt longer than the table
            drv.begin([[1, 2, 3, 4, 5], [1]])
    finally:
        drv.close()
