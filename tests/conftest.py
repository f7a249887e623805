import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


@pytest.fixture(scope="session")
def cuda():
    """Session fixture for GPU tests: fails (does not skip) when the extension or device is missing."""
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    from antares_b200 import _lib
    _lib.load()
    return torch.device("cuda:0")
