import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has = torch.cuda.is_available()
    except Exception:
        has = False
    if has:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


@pytest.fixture(autouse=True, scope="module")
def _no_device_wait_expired(request):
    """After every GPU test module: no bounded device-side wait of the library may have expired
    (cssm_device_error reads and clears the word)."""
    yield
    try:
        import torch
        if not torch.cuda.is_available():
            return
    except Exception:
        return
    import ctypes as C
    from cssm_b200._lib import lib
    torch.cuda.synchronize()
    v = C.c_int(-1)
    assert lib().cssm_device_error(C.byref(v), 1) == 0
    assert v.value == 0, f"device error word {v.value:#x} after {request.module.__name__}"
