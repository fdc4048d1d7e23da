import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a); run with -m gpu on a B200")


@pytest.fixture(scope="session")
def dev():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from spinf_serve_b200 import _lib

    _lib.init(0)
    return torch.device("cuda:0")


@pytest.fixture(autouse=True)
def _device_status_clean(request):
    """after every GPU test the device status word must be clean: a bounded wait that gave up fails the test"""
    yield
    if request.node.get_closest_marker("gpu") is None:
        return
    import torch

    if torch.cuda.is_available():
        from spinf_serve_b200 import _lib

        assert _lib.last_status(raise_on_error=False) == 0
