"""The operator-level C++ tests (tests/cpp/test_ops.cpp): Linear / MatMul created with
Backend::CUDA through the nnops API, pitched TensorViews, stream in ComputeContext.

Two builds of the same source: against the stand-alone API mirror, and -- where the nnops
source tree was available at build time -- against the real nnops headers with nnops' own
operator front end and CPU route linked to this CUDA backend (the drop-in), in which every case
is also compared byte for byte with the reference's CPU result.
"""
import subprocess
from pathlib import Path

import pytest

BIN = Path(__file__).resolve().parent / "cpp" / "_bin"


def test_host_side_builds(nnb200_lib):
    """C++23 host code and the test programs compile and link (no GPU needed)."""
    from nnops_b200.host import build as host_build
    outs = host_build.build_tests()
    assert (BIN / "test_ops_standalone") in outs
    # Without a GPU the program reports that and exits 77 before touching anything.
    import torch
    if not torch.cuda.is_available():
        r = subprocess.run([str(BIN / "test_ops_standalone")], capture_output=True, text=True, timeout=120)
        assert r.returncode == 77, r.stdout + r.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["test_ops_standalone", "test_ops_dropin"])
def test_cpp_operator_tests(cuda_device, name):
    exe = BIN / name
    if not exe.exists():
        if name == "test_ops_dropin":
            pytest.skip("drop-in build needs the nnops source tree at build time")
        from nnops_b200.host import build as host_build
        host_build.build_tests()
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-2000:]
    assert "PASS" in r.stdout
