import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(autouse=True)
def _no_device_side_timeouts(request):
    """After every GPU test: every bounded wait inside the kernels must have completed (status word 0)."""
    yield
    if request.node.get_closest_marker("gpu") is None:
        return
    import ctypes as C
    import torch
    if not torch.cuda.is_available():
        return
    from flashmla_windows_linux_sm120_b200._cabi import lib
    torch.cuda.synchronize()
    st = C.c_int(0)
    rc = lib.fmla_device_status(C.byref(st), 1)
    assert rc == 0 and st.value == 0, f"device status {st.value}: {lib.fmla_last_error_message().decode()}"
