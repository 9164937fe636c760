"""A projection written to disk in the servers' container, uploaded by the library (the reference's upload_w4 step,
server/inference_server_int4_batched.cu:32-45) and run through both GEMV formats, against the oracle."""
import numpy as np
import pytest

import oracle
from blackwell_b200 import synth
from tests.util import max_abs_rel, to_dev

pytestmark = pytest.mark.gpu


def test_uploaded_projection_runs_both_formats(cuda, tmp_path):
    import torch

    from blackwell_b200 import kernels as k
    from blackwell_b200 import weight_files as wf

    M, K, N = 3, 4096, 1000
    packed, sc16, sc32 = synth.int4_weights(N, K, 21)
    prefix = str(tmp_path / "0_self_attn.o_proj")
    wf.write_w4(prefix, packed, sc32)
    w = wf.DeviceW4(prefix)
    try:
        assert (w.K, w.N) == (K, N)
        x32 = synth.activations_f16(M, K, 22).astype(np.float32)
        # reference format: int4 activations, fp32 scales
        xq, xs = oracle.quantize_int4(x32)
        y = torch.empty((M, N), dtype=torch.float32, device="cuda")
        k.gemv_int4_batched(y, to_dev(xq), to_dev(xs), w.packed, w.scale_f32, K, N, M)
        assert max_abs_rel(y.cpu().numpy(), oracle.gemv_w4a4_f64(xq, xs, packed, sc32)) < 2e-5
        # north-star format: int8 activations, binary16 scales (the synthetic scales are binary16 values already,
        # so the conversion at upload is exact)
        x8, x8s = oracle.quantize_int8(x32)
        k.gemv_w4a8(y, to_dev(x8), to_dev(x8s), w.packed, w.scale_f16, K, N, M)
        assert max_abs_rel(y.cpu().numpy(), oracle.gemv_w4a8_f64(x8, x8s, packed, sc16)) < 2e-5
        assert k.device_status() == 0
    finally:
        torch.cuda.synchronize()
        w.close()
