import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def lib():
    """The CUDA library, built if stale (nvcc cross-compiles without a GPU)."""
    from prism_b200 import _lib, build
    build.build()
    return _lib.lib()


@pytest.fixture(scope="session")
def dev(lib):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no GPU")
    return torch.device("cuda", 0)


@pytest.fixture(autouse=True)
def _status_clean(request):
    """After every GPU test the device status word must be clear (no kernel gave up a wait)."""
    yield
    if request.node.get_closest_marker("gpu"):
        import torch
        if torch.cuda.is_available():
            from prism_b200 import _lib
            code, where = _lib.device_status(reset=True)
            assert code == 0, f"device status {code} at {where:#x}"
