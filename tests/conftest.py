import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box with -m gpu)")


@pytest.fixture(scope="session")
def orc():
    from oracle import oracle
    oracle.lib()
    return oracle


@pytest.fixture(scope="session")
def cuda():
    """The CUDA path: native library loaded, torch device available.  Fails (not
    skips) when the extension is missing on a GPU box."""
    import torch
    assert torch.cuda.is_available(), "gpu tests need a CUDA device"
    from deepbind_b200 import _lib
    _lib.load()
    return torch.device("cuda", 0)
