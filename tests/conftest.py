import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "kern-k3_b200"))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
sys.path.insert(0, os.path.join(ROOT, "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


@pytest.fixture(scope="session")
def k3o():
    import k3o as mod
    mod.lib()
    return mod


@pytest.fixture(scope="session")
def k3g():
    """The C-ABI binding; building the library first if this is a fresh checkout."""
    lib = os.path.join(ROOT, "kern-k3_b200", "lib", "libk3g.so")
    if not os.path.exists(lib):
        sys.path.insert(0, os.path.join(ROOT, "kern-k3_b200"))
        import build
        build.build()
    import k3g as mod
    return mod


@pytest.fixture(scope="session")
def dev():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")
