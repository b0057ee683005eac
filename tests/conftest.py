import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "light-tensor_b200", "python")):
    if p not in sys.path:
        sys.path.insert(0, p)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu on the GPU box")


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle package (test infrastructure); builds its C library on first use."""
    import oracle as o
    return o


@pytest.fixture(scope="session")
def golden():
    def load(name):
        return np.load(os.path.join(GOLDEN, name), allow_pickle=False)
    return load


@pytest.fixture(scope="session")
def cuda():
    """torch, after checking that a CUDA device and the built library are really there (no silent skip on the GPU box:
    a missing library is a failure, not a skip)."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import ltq
    ltq.lib()  # raises if libltq.so was not built
    torch.cuda.set_device(0)
    return torch
