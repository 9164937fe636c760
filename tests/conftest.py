import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    # GPU tests fail loudly, never silently skip, when selected with -m gpu on a box without a device;
    # in a plain run on a CPU-only box they are deselected by the marker expression the driver passes.
    pass


@pytest.fixture(scope="session")
def cuda():
    import torch

    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    torch.cuda.set_device(0)
    return torch.device("cuda:0")
