"""Model shapes of the benchmark configurations and the algorithmic byte counts
the roofline figures are computed from."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class ModelShape:
    name: str
    layers: int
    hidden: int
    inter: int
    n_q_heads: int
    n_kv_heads: int
    head_dim: int
    vocab: int
    eps: float = 1e-6

    @property
    def q_dim(self) -> int:
        return self.n_q_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.n_kv_heads * self.head_dim

    def layer_gemvs(self):
        """(name, N, K) of the per-layer projections in the fused form the
        decode step launches: QKV, O, gate+up, down."""
        return [
            ("qkv", self.q_dim + 2 * self.kv_dim, self.hidden),
            ("o", self.hidden, self.q_dim),
            ("gate_up", 2 * self.inter, self.hidden),
            ("down", self.hidden, self.inter),
        ]

    def gemv_set(self):
        """The five matrices of the per-layer GEMV benchmark set."""
        return self.layer_gemvs() + [("lm_head", self.vocab, self.hidden)]


QWEN3_8B = ModelShape("qwen3-8b-shape", 36, 4096, 10944, 32, 8, 128, 151643)
QWEN3_32B = ModelShape("qwen3-32b-shape", 64, 5120, 25600, 64, 8, 128, 151643)


def gemv_bytes(N: int, K: int, M: int, w_scale_bytes: int = 2, x_kind: str = "f16") -> int:
    """Algorithmic bytes of one GEMV call: nibbles + weight scales once,
    activations once, fp32 outputs once.  x_kind: 'f16' (fused quantize),
    'i8' (int8 + f32 block scales), 'i4' (nibbles + f32 block scales), 'f32'."""
    w = N * K // 2 + N * (K // 16) * w_scale_bytes
    if x_kind == "f16":
        x = M * K * 2
    elif x_kind == "f32":
        x = M * K * 4
    elif x_kind == "i8":
        x = M * K + M * (K // 16) * 4
    elif x_kind == "i4":
        x = M * K // 2 + M * (K // 16) * 4
    else:
        raise ValueError(x_kind)
    return w + x + M * N * 4
