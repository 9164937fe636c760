"""Tensor-parallel sharding of the decode GEMVs across the GPUs of one box.

Megatron-style: QKV, gate+up and the LM head are split by output rows (QKV by
whole heads, gate and up by the same row range so SwiGLU stays local); the
O-projection and the down-projection are split along K (on 32-element
boundaries, so every shard keeps the streaming kernel's alignment) and their
partial outputs are summed across ranks.  The only exchanges are therefore an
all-reduce after O and after down, and a gather of the LM-head result.  One
process per GPU; the exchanges go through ``torch.distributed`` (NCCL over
NVLink on the GPU box, gloo in the CPU tests).
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class Shard:
    name: str
    kind: str        # "row" (no exchange), "row_gather" (all-gather of outputs), "k" (all-reduce of partial sums)
    N: int           # full matrix
    K: int
    n0: int          # first output row of this rank (row kinds), else 0
    n_local: int
    k0: int          # first k of this rank (k kind), else 0
    k_local: int
    n_pad: int       # rows per rank in the gathered buffer (row_gather)


def split_even(total_units: int, world: int, rank: int):
    """Contiguous split of ``total_units`` into ``world`` parts differing by at most one unit."""
    base, rem = divmod(total_units, world)
    start = rank * base + min(rank, rem)
    return start, base + (1 if rank < rem else 0)


def shard_rows(name, N, K, world, rank, unit=1, gather=False) -> Shard:
    u0, un = split_even(N // unit, world, rank)
    n0, nl = u0 * unit, un * unit
    if rank == world - 1:
        nl += N % unit
    n_pad = (-(-(N // unit) // world)) * unit + (N % unit)
    return Shard(name, "row_gather" if gather else "row", N, K, n0, nl, 0, K, n_pad)


def shard_k(name, N, K, world, rank, unit=32) -> Shard:
    assert K % unit == 0, (name, K, unit)
    u0, un = split_even(K // unit, world, rank)
    return Shard(name, "k", N, K, 0, N, u0 * unit, un * unit, N)


def shard_gemv_set(mats, world: int, rank: int, head_dim: int = 128):
    """mats: [(name, N, K)] with the names of ``ModelShape.gemv_set``."""
    out = []
    for name, N, K in mats:
        if name == "qkv":
            out.append(shard_rows(name, N, K, world, rank, unit=head_dim))
        elif name == "gate_up":
            out.append(shard_rows(name, N, K, world, rank, unit=2))
        elif name == "lm_head":
            out.append(shard_rows(name, N, K, world, rank, unit=1, gather=True))
        elif name in ("o", "down"):
            out.append(shard_k(name, N, K, world, rank, unit=32))
        else:
            raise ValueError(name)
    return out


class Collectives:
    """The exchanges at the shard boundaries, on the current stream of ``device``.

    ``exchange="nccl"``: ``torch.distributed`` collectives.  ``exchange="peer"``: the K-split partial sums are written
    by the GEMV into a peer-visible slot (``partial_buffer``) and summed by the library's NVLink all-reduce kernel;
    consecutive K-split exchanges must alternate slots, which ``partial_buffer`` does in call order.
    """

    def __init__(self, world: int, rank: int, device, exchange: str = "nccl", slot_floats: int = 0):
        import torch.distributed as dist

        assert exchange in ("nccl", "peer")
        self.world, self.rank, self.device = world, rank, device
        self.dist = dist
        self._gather_buf = {}
        self.peer = None
        self._k = {}          # shard name -> (slot, partial view, result tensor)
        if exchange == "peer":
            from .peer import PeerComm

            self.peer = PeerComm(world, rank, slot_floats, device)
            self.peer.connect_processes()

    def partial_buffer(self, sh: Shard, M: int):
        """The tensor a K-split GEMV of ``sh`` must write to, or None when any tensor will do (NCCL)."""
        if self.peer is None or sh.kind != "k":
            return None
        import torch

        if sh.name not in self._k:
            slot = self.peer.next_slot()
            self._k[sh.name] = (slot, self.peer.slot(slot, M, sh.N),
                                torch.zeros((M, sh.N), dtype=torch.float32, device=self.device))
        return self._k[sh.name][1]

    def finish(self, sh: Shard, y):
        """y: [M, n_local] fp32 (row kinds) or [M, N] partial sums (k kind).  Returns the tensor holding the
        complete result on every rank ([world, M, n_pad] for the gather)."""
        if sh.kind == "k":
            if self.peer is not None:
                slot, part, out = self._k[sh.name]
                assert y.data_ptr() == part.data_ptr(), "the GEMV must write into partial_buffer()"
                self.peer.allreduce(slot, out, out.numel())
                return out
            self.dist.all_reduce(y)
            return y
        if sh.kind == "row_gather":
            import torch

            M = y.shape[0]
            key = (sh.name, M)
            if key not in self._gather_buf:
                self._gather_buf[key] = (
                    torch.zeros((self.world, M, sh.n_pad), dtype=y.dtype, device=y.device),
                    torch.zeros((M, sh.n_pad), dtype=y.dtype, device=y.device))
            full, padded = self._gather_buf[key]
            padded[:, : sh.n_local].copy_(y)
            self.dist.all_gather_into_tensor(full.view(-1), padded.view(-1))
            return full
        return y

    @staticmethod
    def assemble(sh: Shard, full, world: int):
        """[world, M, n_pad] gathered buffer -> [M, N] in row order."""
        import torch

        parts = []
        for r in range(world):
            s = shard_rows(sh.name, sh.N, sh.K, world, r, unit=1, gather=True)
            parts.append(full[r, :, : s.n_local])
        return torch.cat(parts, dim=1)
