"""The allocation-free entry point against the regular one.

nnb200_gemm_i8_static_scratch serves callers that are handed their buffers and must not
allocate device memory themselves (a plugin inside an inference runtime, a latency-critical
loop): its scratch is a fixed array inside the library.  Here it is driven through the C ABI on
two different problems in a row -- the second smaller than the first, so stale contents of the
shared array would show -- and each result must equal, byte for byte, what nnb200_gemm_i8
produces with a caller-provided workspace AND what the CPU oracle computes from the same
bytes.  A batched call and a call that brings the weights' row sums with it (a packed weight)
follow.  Collected last on purpose.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
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
        kw_np = {key: (v.copy() if isinstance(v, np.ndarray) else v) for key, v in kw.items()}
        expect = oracle.gemm_i8(a.cpu().numpy(), w.cpu().numpy(), **kw_np)
        assert np.array_equal(got.cpu().numpy(), expect), "differs from the CPU oracle"


def test_static_scratch_batched_and_packed_row_sums(cuda_device, nnb200_lib):
    """Two more uses of the fixed array: a batch of two (each batch element has its own slice of
    the scratch) and a call whose weight row sums come precomputed from a packed blob."""
    stream = torch.cuda.current_stream(cuda_device).cuda_stream
    rng = np.random.default_rng(11)
    m, n, k = 90, 200, 256
    a = torch.from_numpy(rng.integers(0, 256, (2, m, k), dtype=np.uint8)).to(cuda_device)
    w = torch.from_numpy(rng.integers(-127, 128, (n, k), dtype=np.int8)).to(cuda_device)
    kw = dict(out_kind="s8", out_scale=3.0, out_zp=-3, scale_a=0.02, zp_a=128,
              scale_w=rng.uniform(0.001, 0.02, n).astype(np.float32), zp_w=rng.integers(-9, 10, n).astype(np.int32))
    want = ops.gemm_i8(a, w, **kw)
    got = torch.empty_like(want)
    keep = []
    args = ops.gemm_i8_args(a, w, got, keep=keep, **kw)
    assert args.batch == 2 and args.workspace_bytes > 0
    args.workspace, args.workspace_bytes = None, 0
    capi.check(nnb200_lib.nnb200_gemm_i8_static_scratch(C.byref(args), stream), "static_scratch batch")
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    for b in range(2):
        expect = oracle.gemm_i8(a[b].cpu().numpy(), w.cpu().numpy(), **kw)
        assert np.array_equal(got[b].cpu().numpy(), expect)

    packed = ops.prepack_i8(w, scale_w=kw["scale_w"], zp_w=kw["zp_w"])
    kw2 = dict(kw, scale_w=packed.scale_w, zp_w=packed.zp_w)
    want2 = ops.gemm_i8(a[0], packed.w, r_w=packed.r_w, **kw2)
    got2 = torch.empty_like(want2)
    args = ops.gemm_i8_args(a[0], packed.w, got2, keep=keep, r_w=packed.r_w, **kw2)
    args.workspace, args.workspace_bytes = None, 0
    capi.check(nnb200_lib.nnb200_gemm_i8_static_scratch(C.byref(args), stream), "static_scratch packed")
    torch.cuda.synchronize()
    assert torch.equal(got2, want2)
    assert np.array_equal(got2.cpu().numpy(), oracle.gemm_i8(a[0].cpu().numpy(), w.cpu().numpy(), **kw))


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
