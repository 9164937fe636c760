"""Helpers shared by the tests: numpy <-> device tensors, error metrics."""
import numpy as np


def to_dev(a, device="cuda"):
    import torch

    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).to(device)
    return torch.from_numpy(a).to(device)


def max_abs_rel(y, ref):
    """max_i |y_i - ref_i| / max_i |ref_i| -- the metric the 1e-3 tolerance is stated in."""
    y = np.asarray(y, np.float64)
    ref = np.asarray(ref, np.float64)
    return float(np.max(np.abs(y - ref)) / max(np.max(np.abs(ref)), 1e-30))


TOL = 1e-3  # max-abs-rel tolerance of the fp32 outputs against the high-precision oracle
