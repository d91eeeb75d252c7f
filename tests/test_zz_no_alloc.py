"""The allocation-free entry point against the regular one.

nnb200_gemm_i8_static_scratch serves callers that are handed their buffers and must not
allocate device memory themselves (a plugin inside an inference runtime, a latency-critical
loop): its scratch is a fixed array inside the library.  Here it is driven through the C ABI on
two different problems in a row -- the second smaller than the first, so stale contents of the
shared array would show -- and each result must equal, byte for byte, what nnb200_gemm_i8
produces with a caller-provided workspace.  Collected last on purpose.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from nnops_b200 import capi, ops

pytestmark = pytest.mark.gpu


def _problem(dev, m, n, k, seed, out_kind):
    rng = np.random.default_rng(seed)
    a = torch.from_numpy(rng.integers(0, 256, (m, k), dtype=np.uint8)).to(dev)
    w = torch.from_numpy(rng.integers(-127, 128, (n, k), dtype=np.int8)).to(dev)
    kw = dict(out_kind=out_kind, relu=True, out_scale=2.1, out_zp=4 if out_kind != "s32" else 0,
              bias=rng.integers(-500, 500, n).astype(np.int32),
              scale_a=rng.uniform(0.01, 0.03, m).astype(np.float32),
              scale_w=rng.uniform(0.001, 0.02, n).astype(np.float32),
              zp_a=rng.integers(100, 140, m).astype(np.int32), zp_w=rng.integers(-9, 10, n).astype(np.int32))
    return a, w, kw


def test_static_scratch_matches_workspace_entry(cuda_device, nnb200_lib):
    stream = torch.cuda.current_stream(cuda_device).cuda_stream
    for (m, n, k, seed, kind) in [(300, 520, 512, 1, "s8"), (70, 130, 272, 2, "s32")]:
        a, w, kw = _problem(cuda_device, m, n, k, seed, kind)
        want = ops.gemm_i8(a, w, **kw)                       # regular entry, torch-allocated workspace
        got = torch.empty_like(want)
        keep = []
        args = ops.gemm_i8_args(a, w, got, keep=keep, **kw)
        assert args.workspace_bytes > 0, "the case must need scratch"
        args.workspace = None                               # the new entry point must not need it
        args.workspace_bytes = 0
        capi.check(nnb200_lib.nnb200_gemm_i8_static_scratch(C.byref(args), stream), "static_scratch")
        torch.cuda.synchronize()
        assert torch.equal(got, want)


def test_static_scratch_rejects_oversize(cuda_device, nnb200_lib):
    # 4*(m + n) bytes beyond the fixed array: refused, nothing launched, output untouched.
    m, n, k = 16, capi.STATIC_SCRATCH_BYTES // 4 + 64, 16
    a = torch.zeros((m, k), dtype=torch.int8, device=cuda_device)
    w = torch.zeros((n, k), dtype=torch.int8, device=cuda_device)
    out = torch.full((m, n), 77, dtype=torch.int32, device=cuda_device)
    args = ops.gemm_i8_args(a, w, out, out_kind="s32", zp_a=3, zp_w=1)
    args.workspace = None
    args.workspace_bytes = 0
    before = nnb200_lib.nnb200_launch_count()
    st = nnb200_lib.nnb200_gemm_i8_static_scratch(C.byref(args), torch.cuda.current_stream(cuda_device).cuda_stream)
    assert st == capi.OUT_OF_MEMORY
    assert nnb200_lib.nnb200_launch_count() == before
    torch.cuda.synchronize()
    assert bool((out == 77).all())
