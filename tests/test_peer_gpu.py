"""Peer-memory all-reduce (csrc/peer_allreduce.cu) on two or four GPUs of one box, all driven from this process
(skipped with fewer GPUs), and its bounded wait on one GPU.  The expected value is the fp32 sum in rank order, which the kernel must match bit for
bit on both ranks (all ranks have to hold identical hidden states after the exchange).
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _gpus():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _two_gpus():
    return _gpus() >= 2


@pytest.mark.parametrize("world", [2, 4])
def test_peer_allreduce_ranks_bitwise(world):
    """world 2: the one-step kernel; world 4: the 1.3 MB cases take the two-step (reduce, then store to all) kernel."""
    if _gpus() < world:
        pytest.skip(f"needs {world} GPUs")
    from blackwell_b200.peer import PeerComm

    from blackwell_b200 import kernels as k

    k.set_tuning(10, 256)   # vectors of 256 KiB and more take the two-step kernel on 4+ ranks (default: 4 MiB)
    rows, cols = 64, 5120
    comms = [PeerComm(world, r, rows * cols, torch.device("cuda", r)) for r in range(world)]
    try:
        for r in range(world):
            for q in range(world):
                if q != r:
                    comms[r].attach(comms[q])
        rng = np.random.default_rng(0xB200)
        for it, (m, n) in enumerate([(1, 4096), (64, 5120), (8, 4096), (64, 5120), (3, 5120), (1, 4096)]):
            slot = it & 1
            parts = [rng.standard_normal((m, n)).astype(np.float32) for _ in range(world)]
            resid = rng.standard_normal((m, n)).astype(np.float32) if it % 3 == 0 else None
            outs = []
            for r in range(world):
                dev = torch.device("cuda", r)
                with torch.cuda.device(dev):
                    assert comms[r].next_slot() == slot
                    comms[r].slot(slot, m, n).copy_(torch.from_numpy(parts[r]))
                    outs.append(torch.empty((m, n), dtype=torch.float32, device=dev))
            for r in range(world):   # both kernels are enqueued before either is waited for
                dev = torch.device("cuda", r)
                with torch.cuda.device(dev):
                    res = None if resid is None else torch.from_numpy(resid).to(dev)
                    comms[r].allreduce(slot, outs[r], m * n, residual=res)
            for r in range(world):
                torch.cuda.synchronize(r)
            want = (resid if resid is not None else np.zeros((m, n), np.float32)).copy()
            for r in range(world):
                want = (want + parts[r]).astype(np.float32)
            for r in range(world):
                assert comms[r].status() == 0
                got = outs[r].cpu().numpy()
                assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (it, r)
    finally:
        k.set_tuning(10, 0)
        for r in range(world):
            torch.cuda.synchronize(r)
        for c in comms:
            c.close()


def test_peer_wait_runs_out_and_the_next_call_works():
    """A rank whose peer never calls: the kernel's wait for the peer's flag is bounded (here 5 ms, set through tuning
    key 11), after which it reports status 3, leaves the output untouched and returns -- the context stays usable and
    the next exchange on the same communicator works.  Both communicators live on ONE device (no second GPU needed)
    and only rank 0 ever launches, so no two kernels wait for each other; the peer's part of the second exchange is
    played by the test, which writes the peer's slot and its arrival words directly."""
    import ctypes as C

    from blackwell_b200 import _lib
    from blackwell_b200 import kernels as k
    from blackwell_b200.peer import PeerComm

    assert torch.cuda.is_available()
    dev = torch.device("cuda", 0)
    n = 4096
    c0, c1 = PeerComm(2, 0, n, dev), PeerComm(2, 1, n, dev)
    k.set_tuning(11, 5)
    try:
        c0.attach(c1)
        c1.attach(c0)
        mine = torch.arange(n, dtype=torch.float32, device=dev)
        c0.slot(0, 1, n).copy_(mine.view(1, n))
        out = torch.full((n,), -1.0, dtype=torch.float32, device=dev)
        c0.allreduce(0, out, n)                 # rank 1 never signals
        torch.cuda.synchronize()
        assert c0.status() == 3
        assert c0.status() == 0                 # reading clears it
        assert (out == -1.0).all()              # no result was written
        # second exchange (slot 1, epoch 2 on every CTA): the "peer" has filled its slot and signalled
        c0.slot(1, 1, n).copy_(mine.view(1, n))
        c1.slot(1, 1, n).fill_(0.5)
        L = _lib.load()
        L.bw_peer_comm_slot.restype = C.c_void_p
        base0 = L.bw_peer_comm_slot(c0._h, 0) - 16384        # flags[cta][source rank] at the start of the region

        class _View:
            pass

        v = _View()
        v.__cuda_array_interface__ = {"shape": (160, 8), "typestr": "<i4", "data": (int(base0), False), "version": 2}
        flags = torch.as_tensor(v, device=dev)
        flags[:, 1] = 2
        torch.cuda.synchronize()
        c0.allreduce(1, out, n)
        torch.cuda.synchronize()
        assert c0.status() == 0
        assert torch.equal(out, mine + 0.5)
    finally:
        k.set_tuning(11, 0)
        torch.cuda.synchronize()
        c0.close()
        c1.close()


def test_peer_allreduce_rejects_bad_arguments():
    from blackwell_b200.kernels import KernelError
    from blackwell_b200.peer import PeerComm

    c0 = PeerComm(2, 0, 4096, torch.device("cuda", 0))
    try:
        out = torch.empty(4096, dtype=torch.float32, device="cuda:0")
        with pytest.raises(KernelError):      # the peer was never attached
            c0.allreduce(0, out, 4096)
        with pytest.raises(KernelError):      # larger than a slot
            c0.allreduce(0, out, 8192)
        with pytest.raises(KernelError):      # not a multiple of four floats
            c0.allreduce(0, out, 4094)
    finally:
        c0.close()
