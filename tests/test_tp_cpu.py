"""Tensor-parallel sharding of the GEMV set, world_size 2 over gloo on CPU: every rank computes its shard with the
oracle (standing in for the device kernels), the exchanges of blackwell_b200.tp run over gloo, and each rank must
end with the unsharded result."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from blackwell_b200 import synth, tp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


MATS = [("qkv", 768, 256), ("o", 256, 512), ("gate_up", 1000, 256), ("down", 256, 416), ("lm_head", 1003, 256)]


def _worker(rank, world, port, M):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        coll = tp.Collectives(world, rank, torch.device("cpu"))
        for i, (sh, (name, N, K)) in enumerate(zip(tp.shard_gemv_set(MATS, world, rank), MATS)):
            W, sc16, _ = synth.int4_weights(N, K, 700 + i)
            x = synth.activations_f16(M, K, 800 + i).astype(np.float32)
            full = oracle.gemv_w4a8_f64(*oracle.quantize_int8(x), W, sc16)
            if sh.kind == "k":
                # activations are quantized per 16-block, so a K shard on a 32 boundary quantizes identically
                xs = np.ascontiguousarray(x[:, sh.k0:sh.k0 + sh.k_local])
                Wl = np.ascontiguousarray(W[:, sh.k0 // 2:(sh.k0 + sh.k_local) // 2])
                scl = np.ascontiguousarray(sc16[:, sh.k0 // 16:(sh.k0 + sh.k_local) // 16])
                y = torch.from_numpy(oracle.gemv_w4a8_f64(*oracle.quantize_int8(xs), Wl, scl))
                out = coll.finish(sh, y).numpy()
            else:
                Wl = np.ascontiguousarray(W[sh.n0:sh.n0 + sh.n_local])
                scl = np.ascontiguousarray(sc16[sh.n0:sh.n0 + sh.n_local])
                y = torch.from_numpy(oracle.gemv_w4a8_f64(*oracle.quantize_int8(x), Wl, scl))
                res = coll.finish(sh, y)
                if sh.kind == "row_gather":
                    out = tp.Collectives.assemble(sh, res, world).numpy()
                else:
                    out = None
                    assert np.allclose(res.numpy(), full[:, sh.n0:sh.n0 + sh.n_local], rtol=1e-12)
            if out is not None:
                assert out.shape == full.shape
                assert np.allclose(out, full, rtol=1e-9, atol=1e-12), name
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("M", [1, 3])
def test_sharded_gemv_set_world2_gloo(M):
    mp.spawn(_worker, args=(2, _free_port(), M), nprocs=2, join=True)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_shard_plan_covers_everything(world):
    from blackwell_b200 import shapes

    for shape in (shapes.QWEN3_8B, shapes.QWEN3_32B):
        mats = shape.gemv_set()
        for name, N, K in mats:
            rows, ks = 0, 0
            for r in range(world):
                sh = [s for s in tp.shard_gemv_set(mats, world, r) if s.name == name][0]
                if sh.kind == "k":
                    assert sh.k0 == ks and sh.k_local % 32 == 0 and sh.n_local == N
                    ks += sh.k_local
                else:
                    assert sh.n0 == rows and sh.k_local == K and sh.n_local <= sh.n_pad
                    rows += sh.n_local
            assert (ks == K) if name in ("o", "down") else (rows == N)
