import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


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
def _no_device_side_timeouts(request):
    """After every GPU test: no bounded device-side wait may have run out."""
    yield
    if "gpu" in request.keywords:
        import torch
        if torch.cuda.is_available():
            from sla_b200 import _lib
            code = _lib.poll_device_error(clear=True)
            assert code == 0, f"a tcgen05 kernel reported a timed-out wait (code {code})"
