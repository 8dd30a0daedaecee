import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100); run with -m gpu")


def _has_gpu():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def native_lib():
    """The in-tree native library, built on demand (nvcc cross-compiles without a GPU)."""
    from flextensor_b200 import build as ftb_build, backend
    ftb_build.build()
    return backend.lib()


@pytest.fixture(scope="session")
def c_oracle():
    from oracle import c_oracle as co
    co.lib()
    return co


GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")
