"""Seeded synthetic inputs with the benchmark's shapes and value distributions.

They stand in for real Qwen3 weights (not available offline).  Host versions
(numpy, PCG64) feed both the oracle and the device path in the parity tests; the
``*_device`` versions fill large benchmark buffers directly in HBM with torch's
generator.

Distributions: weights are int4 symmetric integers uniform in [-7, 7] stored as
offset-binary nibbles (q + 8), two per byte along K, even k in the low nibble;
one binary16 scale per 16-element k-block drawn as |N(0, 0.02)| + 1e-3 (the fp32
copy used by the reference-format path is the same value widened);
activations are binary16 N(0, 1); norm weights 1 + 0.1 N(0, 1).
"""
from __future__ import annotations

import numpy as np

SEED_BASE = 0xB2000000


def rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(SEED_BASE + int(seed)))


def int4_weights(N: int, K: int, seed: int, full_range: bool = False):
    """-> (W_packed u8 [N][K/2], scale_f16 [N][K/16], scale_f32 [N][K/16]).
    ``full_range`` also emits nibble 0 (q = -8), which real weight files never
    hold but the kernels must decode."""
    g = rng(seed)
    lo, hi = (-8, 8) if full_range else (-7, 8)
    q = g.integers(lo, hi, size=(N, K), dtype=np.int8)
    nib = (q + 8).astype(np.uint8)
    packed = (nib[:, 0::2] | (nib[:, 1::2] << 4)).astype(np.uint8)
    sc = (np.abs(g.normal(0.0, 0.02, size=(N, K // 16))) + 1e-3).astype(np.float16)
    return np.ascontiguousarray(packed), sc, sc.astype(np.float32)


def activations_f16(M: int, K: int, seed: int) -> np.ndarray:
    return rng(seed).normal(0.0, 1.0, size=(M, K)).astype(np.float16)


def norm_weight(H: int, seed: int) -> np.ndarray:
    return (1.0 + 0.1 * rng(seed).normal(0.0, 1.0, size=H)).astype(np.float32)


def kv_cache_f16(shape, seed: int) -> np.ndarray:
    return rng(seed).normal(0.0, 1.0, size=shape).astype(np.float16)


# ---------------------------------------------------------------- device side
def int4_weights_device(N: int, K: int, seed: int, device="cuda", scale_dtype=None):
    """Same distributions, generated in HBM: (W_packed u8, scale f16 or f32)."""
    import torch

    gen = torch.Generator(device=device)
    gen.manual_seed(SEED_BASE + int(seed))
    lo = torch.randint(1, 16, (N, K // 2), dtype=torch.uint8, device=device, generator=gen)
    hi = torch.randint(1, 16, (N, K // 2), dtype=torch.uint8, device=device, generator=gen)
    packed = lo | (hi << 4)
    del lo, hi
    sc = torch.empty((N, K // 16), dtype=torch.float32, device=device)
    sc.normal_(0.0, 0.02, generator=gen)
    sc = sc.abs_().add_(1e-3).to(torch.float16)
    if scale_dtype is not None and scale_dtype != torch.float16:
        sc = sc.to(scale_dtype)
    return packed, sc


def activations_f16_device(M: int, K: int, seed: int, device="cuda"):
    import torch

    gen = torch.Generator(device=device)
    gen.manual_seed(SEED_BASE + int(seed))
    x = torch.empty((M, K), dtype=torch.float32, device=device)
    x.normal_(0.0, 1.0, generator=gen)
    return x.to(torch.float16)
