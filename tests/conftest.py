"""Test configuration: registers the ``gpu`` marker and skips GPU tests when no device is present."""

import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200) and the built kernel library")
    config.addinivalue_line("markers", "slow: long-running test")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _kernel_status_guard(request):
    """After every GPU test, fail if a kernel reported that one of its bounded waits ran out."""
    yield
    if "gpu" in request.keywords:
        import torch

        if torch.cuda.is_available():
            from easydel_b200.ops import _lib

            if _lib.available():
                _lib.check_status()
