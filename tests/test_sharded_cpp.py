"""The C++ sharded layer (include/nnops_b200/sharded_linear.hpp) through its forked-ranks test
program (tests/cpp/test_sharded.cpp).

CPU: the host-side exchange the ranks use for IPC handles and for "is everyone still there?" --
including a rank that announces its leaving and one that never joins.  A lost rank is made on
the host only; no GPU is faulted or hung to test this.
GPU: one rank per GPU (as many as the box has, up to four); every rank's full output must be
byte-identical to the single-GPU GEMM over the whole weight.
"""
import subprocess
from pathlib import Path

import pytest

BIN = Path(__file__).resolve().parent / "cpp" / "_bin" / "test_sharded"


def _exe() -> Path:
    if not BIN.exists():
        from nnops_b200.host import build as host_build
        host_build.build_tests()
    return BIN


def test_exchange_and_lost_ranks_on_the_host(nnb200_lib):
    r = subprocess.run([str(_exe()), "--exchange"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "PASS" in r.stdout
    for line in ("4 ranks x 300 steps: ok", "a rank leaves between steps: ok", "a rank never joins: ok"):
        assert line in r.stdout


@pytest.mark.gpu
def test_cpp_sharded_layer_matches_single_gpu(cuda_device):
    import torch
    world = min(torch.cuda.device_count(), 4)
    if world == 3:
        world = 2
    r = subprocess.run([str(_exe()), "--gpus", str(world)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert f"PASS: {world} ranks" in r.stdout
