"""The allocation-free attention entry point against the allocating one.

Some hosts of the library may not call the CUDA allocator while they serve (all device memory already belongs
to their own pool, or allocation is switched off after start-up); for them
bw_attention_decode_batched_gqa_noalloc keeps its split partials in a fixed array inside the library.  The test
calls it through the C ABI twice in a row -- the second call on a different, shorter problem, so anything left
in the shared array by the first call would show -- and compares each result with the existing entry point on
the same inputs, with the tolerance the other attention tests use.  It also checks that a problem too large for
the fixed array is refused.  The file sorts last so that a run stopping at the first failure has already run
every other test.
"""
import numpy as np
import pytest

from blackwell_b200 import synth
from tests.util import max_abs_rel, to_dev

pytestmark = pytest.mark.gpu


def _case(k, M, nqh, nkv, max_seq, pos, seed):
    import torch

    hd = 128
    g = synth.rng(seed)
    Q = to_dev(g.normal(size=(M, nqh * hd)).astype(np.float32))
    kv_batch = nkv * max_seq * hd
    Kc = to_dev(g.normal(size=M * kv_batch).astype(np.float32))
    Vc = to_dev(g.normal(size=M * kv_batch).astype(np.float32))
    d_pos = to_dev(np.array([pos], np.int32))
    ref = torch.empty((M, nqh * hd), dtype=torch.float32, device="cuda")
    out = torch.full_like(ref, float("nan"))
    k.attention_decode_batched_gqa_device(ref, Q, Kc, Vc, d_pos, nqh, nkv, hd, max_seq, M, kv_batch, 0)
    k.attention_decode_batched_gqa_noalloc(out, Q, Kc, Vc, d_pos, nqh, nkv, hd, max_seq, M, kv_batch, 0)
    torch.cuda.synchronize()
    assert torch.isfinite(out).all()
    assert max_abs_rel(out.cpu().numpy(), ref.cpu().numpy()) < 1e-4


def test_noalloc_attention_matches_allocating_entry_point_twice(cuda):
    from blackwell_b200 import kernels as k

    _case(k, M=2, nqh=32, nkv=8, max_seq=2048, pos=1900, seed=301)   # many splits, long context
    _case(k, M=3, nqh=16, nkv=8, max_seq=512, pos=37, seed=302)      # fewer, mostly empty splits


def test_noalloc_attention_refuses_what_does_not_fit(cuda):
    import torch

    from blackwell_b200 import kernels as k
    from blackwell_b200.kernels import CUDA_ERROR_INVALID_VALUE, KernelError

    # 32 sequences x 64 heads x 2 splits x 130 floats = 532,480 floats > the 524,288 of the fixed array (the
    # split count follows the SM count: 2 on a 148-SM B200).  The check comes before any launch, so the cache
    # pointers are never touched.
    if torch.cuda.get_device_properties(0).multi_processor_count != 148:
        pytest.skip("the refused size is derived for a 148-SM device")
    M, nqh, nkv, hd, max_seq = 32, 64, 8, 128, 128
    # real, fully sized buffers: were the call ever accepted it would still read only memory it was given
    t = torch.zeros(M * nqh * hd, dtype=torch.float32, device="cuda")
    kv = torch.zeros(M * nkv * max_seq * hd, dtype=torch.float32, device="cuda")
    with pytest.raises(KernelError) as e:
        k.attention_decode_batched_gqa_noalloc(t, t, kv, kv, to_dev(np.array([0], np.int32)), nqh, nkv, hd,
                                               max_seq, M, nkv * max_seq * hd, 0)
    assert e.value.code == CUDA_ERROR_INVALID_VALUE
