import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


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
def golden_tests():
    """Outputs of the reference's own torch reference functions (tests/golden/make_golden_from_reference_tests.py)."""
    return np.load(os.path.join(ROOT, "tests", "golden", "reference_tests.npz"))


@pytest.fixture(scope="session")
def golden_cuda():
    """Outputs of the reference's own CUDA kernels on a B200 (tests/golden/capture_reference_cuda_kernels.py)."""
    return np.load(os.path.join(ROOT, "tests", "golden", "reference_cuda_kernels.npz"))


@pytest.fixture(scope="session")
def flib():
    from fluke_b200 import lib
    return lib.load()


@pytest.fixture(autouse=True)
def _device_status_clean(request):
    """After every GPU test the device status word must be clear (no bounded wait gave up)."""
    yield
    if "gpu" in request.keywords and _has_gpu():
        import torch
        from fluke_b200 import lib
        torch.cuda.synchronize()
        assert lib.read_status() == 0, "a device-side wait timed out"
