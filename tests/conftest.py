import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _device_status_clean(request):
    """After every GPU test the device status word must be zero (no bounded wait ran out)."""
    yield
    if "gpu" in request.keywords:
        import torch

        if torch.cuda.is_available():
            from b200fw import _native as nv

            assert nv.read_status() == 0, "a kernel recorded an error status"
