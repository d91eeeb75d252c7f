"""The bounded pipeline waits: a wait nothing satisfies must run out, leave a code the host can
read, and leave the context usable.  The failure is a barrier that nothing arrives at -- no
fault, trap or endless loop is involved."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_wait_runs_out_and_context_survives(nnb200_lib):
    from nnops_b200 import capi, ops
    import oracle

    dev = torch.device("cuda:0")
    assert capi.take_device_error() == 0
    stream = torch.cuda.current_stream(dev).cuda_stream

    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    capi.selftest_wait_limit(2_000_000, stream)          # about 1 ms at ~2 GHz
    stop.record()
    torch.cuda.synchronize(dev)
    assert start.elapsed_time(stop) < 200.0              # it gave up; it did not hang
    assert capi.take_device_error() == capi.DEVICE_ERROR_SELFTEST
    assert capi.take_device_error() == 0                 # reading clears the word

    # The context is intact: a tensor-core GEMM right after is still bit-exact.
    g = torch.Generator().manual_seed(7)
    a = torch.randint(-128, 128, (128, 256), dtype=torch.int8, generator=g)
    w = torch.randint(-128, 128, (256, 256), dtype=torch.int8, generator=g)
    y = ops.gemm_i8(a.to(dev), w.to(dev), out_kind="s32")
    want = oracle.gemm_i8(a.numpy(), w.numpy(), out_kind="s32")
    assert (y.cpu().numpy() == want).all()
    assert capi.take_device_error() == 0


def test_wait_limit_argument_checked(nnb200_lib):
    from nnops_b200 import capi

    for bad in (0, -5, 10**12):
        with pytest.raises(capi.Nnb200Error):
            capi.selftest_wait_limit(bad, None)
    assert capi.take_device_error() == 0
