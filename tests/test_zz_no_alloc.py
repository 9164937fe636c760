"""The allocation-free attention entry point against the CPU oracle and against the allocating one.

Some hosts of the library may not call the CUDA allocator while they serve (all device memory already belongs
to their own pool, or allocation is switched off after start-up); for them
bw_attention_decode_batched_gqa_noalloc keeps its split partials in a fixed array inside the library.  The test
calls it through the C ABI twice in a row -- the second call on a different, shorter problem, so anything left
in the shared array by the first call would show -- and compares each result with the CPU oracle and with the
existing entry point on the same inputs, with the tolerance the other attention tests use.  It also checks that a problem too large for
the fixed array is refused.  The file sorts last so that a run stopping at the first failure has already run
every other test.
"""
import numpy as np
import pytest

import oracle
from blackwell_b200 import synth
from tests.util import max_abs_rel, to_dev

pytestmark = pytest.mark.gpu


def _case(k, M, nqh, nkv, max_seq, pos, seed):
    import torch

    hd = 128
    g = synth.rng(seed)
    Qh = g.normal(size=(M, nqh * hd)).astype(np.float32)
    kv_batch = nkv * max_seq * hd
    Kh = g.normal(size=M * kv_batch).astype(np.float32)
    Vh = g.normal(size=M * kv_batch).astype(np.float32)
    Q, Kc, Vc = to_dev(Qh), to_dev(Kh), to_dev(Vh)
    d_pos = to_dev(np.array([pos], np.int32))
    ref = torch.empty((M, nqh * hd), dtype=torch.float32, device="cuda")
    out = torch.full_like(ref, float("nan"))
    k.attention_decode_batched_gqa_device(ref, Q, Kc, Vc, d_pos, nqh, nkv, hd, max_seq, M, kv_batch, 0)
    k.attention_decode_batched_gqa_noalloc(out, Q, Kc, Vc, d_pos, nqh, nkv, hd, max_seq, M, kv_batch, 0)
    torch.cuda.synchronize()
    assert torch.isfinite(out).all()
    assert max_abs_rel(out.cpu().numpy(), ref.cpu().numpy()) < 1e-4
    cpu = oracle.attention_decode_gqa(Qh, Kh, Vh, pos, nqh, nkv, hd, max_seq, M, kv_batch, 0)
    assert max_abs_rel(out.cpu().numpy(), cpu) < 1e-4


def test_noalloc_attention_matches_allocating_entry_point_twice(cuda):
    from blackwell_b200 import kernels as k

    _case(k, M=2, nqh=32, nkv=8, max_seq=2048, pos=1900, seed=301)   # many splits, long context
    _case(k, M=3, nqh=16, nkv=8, max_seq=512, pos=37, seed=302)      # fewer, mostly empty splits


def test_noalloc_attention_refuses_what_does_not_fit(cuda):
    import torch

    from blackwell_b200 import kernels as k
    from blackwell_b200.kernels import CUDA_ERROR_INVALID_VALUE, KernelError

    # The split count follows the SM count (about two CTAs per SM over the (sequence, kv head) pairs, at least 64
    # positions per split, at most 64 splits); pick the smallest batch whose partial records -- sequences x heads x
    # splits x 130 floats -- exceed the 524,288 floats of the fixed array.  The check comes before any launch, so
    # the cache contents are never read.
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    nqh, nkv, hd, max_seq = 64, 8, 128, 128

    def floats_needed(M):
        nsplit = max(1, min((2 * sms + M * nkv - 1) // (M * nkv), (max_seq + 63) // 64, 64))
        split_len = -(-max_seq // nsplit)
        split_len = -(-split_len // 4) * 4
        nsplit = -(-max_seq // split_len)
        return M * nqh * nsplit * 130 if nsplit > 1 else 0

    M = next((m for m in range(1, 257) if floats_needed(m) > (1 << 19)), None)
    if M is None:
        pytest.skip("no batch up to 256 overflows the fixed array on this device")
    # real, fully sized buffers: were the call ever accepted it would still read only memory it was given
    t = torch.zeros(M * nqh * hd, dtype=torch.float32, device="cuda")
    kv = torch.zeros(M * nkv * max_seq * hd, dtype=torch.float32, device="cuda")
    with pytest.raises(KernelError) as e:
        k.attention_decode_batched_gqa_noalloc(t, t, kv, kv, to_dev(np.array([0], np.int32)), nqh, nkv, hd,
                                               max_seq, M, nkv * max_seq * hd, 0)
    assert e.value.code == CUDA_ERROR_INVALID_VALUE
