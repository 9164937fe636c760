"""Generates the fixtures tests/golden/ref_*.npz from the reference's own CUDA
kernels (oracle/_ref/libblackwell_ref.so, built by `make -C oracle ref` from the
reference sources, unchanged, for sm_100a).  Needs a GPU:

    python -m tests.golden.make_golden [outdir]

Inputs are derived from seeds (blackwell_b200.synth), so only the reference's
outputs are stored.  The CPU test test_oracle_cpu.py re-creates the inputs, runs
the oracle and compares; this is what pins the oracle to the reference.
"""
import os
import sys

import numpy as np

from blackwell_b200 import synth

# name -> (M, K, N, seed); kept small so the fixtures stay a few KB each.
CASES = {
    "m1_k4096_n64": dict(M=1, K=4096, N=64, seed=101),
    "m3_k1040_n48": dict(M=3, K=1040, N=48, seed=102),   # K = 16 * 65 (odd block count, tail lanes)
    "m16_k512_n32": dict(M=16, K=512, N=32, seed=103),   # the reference's maximum batch
    "m2_k10944_n16": dict(M=2, K=10944, N=16, seed=104), # the down-projection K
}


def make_inputs(case):
    M, K, N, seed = case["M"], case["K"], case["N"], case["seed"]
    W, sc16, sc32 = synth.int4_weights(N, K, seed, full_range=True)
    x16 = synth.activations_f16(M, K, seed + 1000)
    x32 = x16.astype(np.float32)
    if M > 1:
        x32[1, :16] = 0.0          # an all-zero block: degenerate scale rule
        x32[1, 16:32] *= 1e-12     # below the 1e-10 threshold
    return dict(W=W, sc16=sc16, sc32=sc32, x32=x32, nw=synth.norm_weight(K, seed + 2000))


def attn_inputs(case):
    g = synth.rng(case["seed"] + 3000)
    nqh, nkv, hd, max_seq, M, pos = 8, 2, 128, 96, 2, 70
    layer_off = nkv * max_seq * hd
    kv_batch = 2 * layer_off
    return dict(Q=g.normal(size=(M, nqh * hd)).astype(np.float32),
                Kc=g.normal(size=(M * kv_batch)).astype(np.float32),
                Vc=g.normal(size=(M * kv_batch)).astype(np.float32),
                nqh=nqh, nkv=nkv, max_seq=max_seq, M=M, pos=pos, kv_batch=kv_batch, layer_off=layer_off)


def main(outdir):
    import torch

    from oracle import ref_cuda as ref

    assert torch.cuda.is_available() and ref.available()
    dev = "cuda"
    os.makedirs(outdir, exist_ok=True)
    for name, case in CASES.items():
        M, K, N = case["M"], case["K"], case["N"]
        inp = make_inputs(case)
        x = torch.from_numpy(inp["x32"]).to(dev)
        W = torch.from_numpy(inp["W"]).to(dev)
        sc = torch.from_numpy(inp["sc32"]).to(dev)
        q4 = torch.empty((M, K // 2), dtype=torch.uint8, device=dev)
        s4 = torch.empty((M, K // 16), dtype=torch.float32, device=dev)
        ref.quantize_int4_batched(q4, s4, x, K, M)
        q8 = torch.empty((M, K), dtype=torch.int8, device=dev)
        s8 = torch.empty((M * K // 16,), dtype=torch.float32, device=dev)
        ref.quantize_int8(q8, s8, x, M * K)
        y = torch.empty((M, N), dtype=torch.float32, device=dev)
        ref.gemv_int4_batched(y, q4, s4, W, sc, K, N, M)
        out = dict(case=name, q4=q4.cpu().numpy(), s4=s4.cpu().numpy(), q8=q8.cpu().numpy(), s8=s8.cpu().numpy(),
                   y_w4a4=y.cpu().numpy())
        if K <= 4096:  # the reference RMSNorm drops elements >= 4096
            nw = torch.from_numpy(inp["nw"]).to(dev)
            r = torch.empty_like(x)
            ref.fused_rmsnorm_batched(r, x, nw, K, 1e-6, M)
            out["rms"] = r.cpu().numpy()
        sw = torch.empty((K,), dtype=torch.float32, device=dev)
        ref.apply_swiglu(sw, x[0], x[-1], K)
        out["swiglu"] = sw.cpu().numpy()
        am = torch.empty((1,), dtype=torch.int32, device=dev)
        ref.sample_argmax_gpu(y[0], N, am)
        out["argmax"] = am.cpu().numpy()[0]
        if name == "m1_k4096_n64":
            a = attn_inputs(case)
            Q = torch.from_numpy(a["Q"]).to(dev)
            Kc = torch.from_numpy(a["Kc"]).to(dev)
            Vc = torch.from_numpy(a["Vc"]).to(dev)
            o = torch.empty_like(Q)
            # per-sequence launches: the batched kernel's softmax is racy across warps for M > 1 long contexts
            ref.attention_decode_batched_gqa(o, Q, Kc, Vc, a["pos"], a["nqh"], a["nkv"], 128, a["max_seq"], a["M"],
                                             a["kv_batch"], a["layer_off"])
            out["attn"] = o.cpu().numpy()
        torch.cuda.synchronize()
        np.savez_compressed(os.path.join(outdir, f"ref_{name}.npz"), **out)
        print("wrote", name)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.dirname(os.path.abspath(__file__)))
