import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    config.addinivalue_line("markers", "expects_wait_timeout: the test makes a bounded device-side wait run out on purpose")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


@pytest.fixture(autouse=True)
def _no_device_side_give_up(request):
    """After every GPU test: no bounded wait inside a kernel may have given up (a give-up leaves a
    launch's outputs invalid without any error on the host side)."""
    yield
    if request.node.get_closest_marker("gpu") is None or request.node.get_closest_marker("expects_wait_timeout"):
        return
    import torch
    if not torch.cuda.is_available():
        return
    from mamba_b200 import _lib
    for d in range(torch.cuda.device_count()):
        assert _lib.device_status(d) == 0, f"a kernel's bounded wait gave up on cuda:{d} during {request.node.name}"
