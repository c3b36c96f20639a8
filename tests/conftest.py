import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def native():
    """Builds (if needed) and loads libtsb200.so."""
    from seq2seqsharp_b200 import _native, build
    build.build()
    return _native.lib()


@pytest.fixture(scope="session")
def oracle():
    from oracle import cpu_oracle
    cpu_oracle.lib()
    return cpu_oracle


@pytest.fixture(scope="session")
def cuda(native):
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a GPU test was selected but no CUDA device is visible (there is no CPU fallback)")
    torch.cuda.set_device(0)
    return torch.device("cuda:0")
