import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.build()
    return O


@pytest.fixture(scope="session")
def btm():
    """The loaded C ABI plus torch device plumbing; GPU tests only."""
    import torch
    from beantensor_b200 import _lib, ops
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    L = _lib.lib()  # raises if libbtm.so is missing: no fallback exists
    ops.init(0)
    return ops
