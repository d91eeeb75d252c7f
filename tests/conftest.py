import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def nnb200_lib():
    """The built C-ABI library; building is cheap when it is up to date."""
    from nnops_b200 import build, capi
    build.build()
    return capi.lib()


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


@pytest.fixture(autouse=True)
def _no_device_error(request):
    """After every GPU test: no kernel may have recorded a pipeline-timeout code."""
    yield
    if request.node.get_closest_marker("gpu") is not None:
        from nnops_b200 import capi
        assert capi.take_device_error() == 0


@pytest.fixture
def knobs(nnb200_lib):
    """Set measurement switches of the library for one test; every one is restored afterwards."""
    from nnops_b200 import capi
    saved = {}

    def set_(name, value):
        prev = capi.set_knob(name, value)
        saved.setdefault(name, prev)

    yield set_
    for name, prev in saved.items():
        capi.set_knob(name, prev)
