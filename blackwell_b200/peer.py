"""Peer-memory all-reduce for the tensor-parallel decode step (host side of ``csrc/peer_allreduce.cu``).

One ``PeerComm`` per rank.  Between processes (``torchrun``) the 64-byte CUDA IPC handles travel through
``torch.distributed``; inside one process two communicators on two devices are attached to each other directly.
The K-split GEMV writes into ``next_slot()`` and ``allreduce`` sums that slot across ranks into a local tensor.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from .kernels import KernelError, _p, _s

_L = _lib.load()
_L.bw_peer_comm_slot.restype = C.c_void_p
_L.bw_peer_comm_slot.argtypes = [C.c_void_p, C.c_int]
_L.bw_peer_comm_create.argtypes = [C.c_int, C.c_int, C.c_size_t, C.POINTER(C.c_void_p)]
_L.bw_peer_comm_handle.argtypes = [C.c_void_p, C.c_void_p]
_L.bw_peer_comm_open.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
_L.bw_peer_comm_attach.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
_L.bw_peer_allreduce_f32.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
_L.bw_peer_comm_status.argtypes = [C.c_void_p, C.POINTER(C.c_int)]
_L.bw_peer_comm_destroy.argtypes = [C.c_void_p]


def _chk(name, code):
    if code != 0:
        raise KernelError(name, code)


class PeerComm:
    def __init__(self, world: int, rank: int, slot_floats: int, device):
        self.world, self.rank, self.device = world, rank, torch.device(device)
        self.slot_floats = int(slot_floats)
        self._turn = 0
        h = C.c_void_p()
        with torch.cuda.device(self.device):
            _chk("peer_comm_create", _L.bw_peer_comm_create(world, rank, self.slot_floats * 4, C.byref(h)))
        self._h = h

    # ---- wiring
    def connect_processes(self):
        """Exchanges IPC handles with the other ranks of the default process group (one process per GPU)."""
        import torch.distributed as dist

        raw = (C.c_ubyte * 64)()
        _chk("peer_comm_handle", _L.bw_peer_comm_handle(self._h, raw))
        mine = torch.tensor(list(raw), dtype=torch.uint8, device=self.device)
        allh = torch.empty((self.world, 64), dtype=torch.uint8, device=self.device)
        dist.all_gather_into_tensor(allh.view(-1), mine)
        allh = allh.cpu()
        with torch.cuda.device(self.device):
            for r in range(self.world):
                if r != self.rank:
                    buf = (C.c_ubyte * 64)(*allh[r].tolist())
                    _chk("peer_comm_open", _L.bw_peer_comm_open(self._h, r, buf))
        dist.barrier()

    def attach(self, other: "PeerComm"):
        """Same-process wiring (tests): makes ``other``'s region visible to this communicator."""
        _chk("peer_comm_attach", _L.bw_peer_comm_attach(self._h, other.rank, other._h))

    # ---- use
    def slot(self, slot: int, rows: int, cols: int) -> torch.Tensor:
        """A [rows, cols] fp32 view of one of the two local slots (memory owned by the communicator)."""
        assert rows * cols <= self.slot_floats
        ptr = _L.bw_peer_comm_slot(self._h, slot)
        n = rows * cols

        class _Holder:  # __cuda_array_interface__ view of library-owned memory
            pass

        hld = _Holder()
        hld.__cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (int(ptr), False), "version": 2}
        with torch.cuda.device(self.device):
            t = torch.as_tensor(hld, device=self.device)
        return t.view(rows, cols)

    def next_slot(self) -> int:
        s = self._turn & 1
        self._turn += 1
        return s

    def allreduce(self, slot: int, out: torch.Tensor, n: int, residual: torch.Tensor | None = None, stream=None):
        _chk("peer_allreduce_f32", _L.bw_peer_allreduce_f32(self._h, slot, _p(out), _p(residual), n, _s(stream)))

    def status(self) -> int:
        v = C.c_int(0)
        with torch.cuda.device(self.device):
            _chk("peer_comm_status", _L.bw_peer_comm_status(self._h, C.byref(v)))
        return v.value

    def close(self):
        if self._h:
            with torch.cuda.device(self.device):
                _L.bw_peer_comm_destroy(self._h)
            self._h = None
