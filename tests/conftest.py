import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200) and the native library")
    config.addinivalue_line("markers", "expects_status: the test makes a bounded device wait run out on purpose "
                                       "and checks the status words itself")


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda", 0)


@pytest.fixture(autouse=True)
def _check_device_status(request):
    """After every GPU test make sure no kernel recorded a timeout/abort status."""
    yield
    if request.node.get_closest_marker("gpu") is None:
        return
    if request.node.get_closest_marker("expects_status") is not None:
        return
    import torch
    if torch.cuda.is_available():
        from gpt_from_scratch_b200.ops import _lib
        code, detail = _lib.read_status(clear=True)
        assert code == 0, f"device status {code}: {_lib.STATUS_NAMES.get(code)} detail=0x{detail:x}"
