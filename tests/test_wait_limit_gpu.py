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


def _flag_arrays(dev, count):
    import ctypes as C
    from nnops_b200 import capi
    arrays = [torch.zeros(capi.RANK_FLAG_BYTES // 4, dtype=torch.int32, device=dev) for _ in range(count)]
    table = (C.c_void_p * count)(*[t.data_ptr() for t in arrays])
    return arrays, table


def test_rank_barrier_protocol_on_one_gpu(nnb200_lib):
    """The device-side rank barrier, two ranks' flag arrays on one GPU, launches strictly one
    after the other (kernels that wait for each other never run side by side on one GPU):
    rank 1 announces epoch 1 and, with nobody answering, gives up after a millisecond with code
    8; rank 0 then finds rank 1's epoch already there and passes at once; so does rank 1's
    second call, because rank 0 is now one epoch ahead of what it needs."""
    from nnops_b200 import capi

    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream(dev).cuda_stream
    arrays, table = _flag_arrays(dev, 2)
    lib = capi.lib()
    short = 2_000_000

    capi.check(lib.nnb200_rank_barrier(table, 2, 1, short, stream), "nnb200_rank_barrier")
    assert capi.take_device_error() == capi.DEVICE_ERROR_PEER_WAIT
    assert arrays[0][1].item() == 1 and arrays[1][8].item() == 1     # announced at rank 0; own epoch advanced

    capi.check(lib.nnb200_rank_barrier(table, 2, 0, short, stream), "nnb200_rank_barrier")
    assert capi.take_device_error() == 0
    assert arrays[1][0].item() == 1 and arrays[0][8].item() == 1

    capi.check(lib.nnb200_rank_barrier(table, 2, 0, short, stream), "nnb200_rank_barrier")   # rank 0: epoch 2, alone
    assert capi.take_device_error() == capi.DEVICE_ERROR_PEER_WAIT
    capi.check(lib.nnb200_rank_barrier(table, 2, 1, short, stream), "nnb200_rank_barrier")   # rank 1: epoch 2, answered
    assert capi.take_device_error() == 0

    # A world of one has nobody to wait for.
    solo, solo_table = _flag_arrays(dev, 1)
    capi.check(lib.nnb200_rank_barrier(solo_table, 1, 0, short, stream), "nnb200_rank_barrier")
    assert capi.take_device_error() == 0 and solo[0][8].item() == 1


def test_rank_barrier_timeout_is_sticky_on_the_host(nnb200_lib):
    """A barrier that ran out of time must not pass silently: until the error word has been
    read, the next barrier and the next sharded GEMM on the device are refused on the host,
    with nothing launched."""
    import ctypes as C
    from nnops_b200 import capi, ops

    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream(dev).cuda_stream
    arrays, table = _flag_arrays(dev, 2)
    lib = capi.lib()
    assert capi.take_device_error() == 0
    capi.check(lib.nnb200_rank_barrier(table, 2, 0, 2_000_000, stream), "nnb200_rank_barrier")   # nobody answers
    torch.cuda.synchronize(dev)
    before = lib.nnb200_launch_count()
    assert lib.nnb200_rank_barrier(table, 2, 0, 2_000_000, stream) == capi.INTERNAL
    a = torch.zeros((256, 256), dtype=torch.int8, device=dev)
    w = torch.zeros((256, 256), dtype=torch.int8, device=dev)
    out = torch.full((256, 512), 9, dtype=torch.int8, device=dev)
    other = torch.full((256, 512), 9, dtype=torch.int8, device=dev)
    args = ops.gemm_i8_args(a, w, out[:, :256], out_kind="s8")
    args.num_peer_outs = 1
    args.peer_out[0] = other.data_ptr()
    assert lib.nnb200_gemm_i8(C.byref(args), stream) == capi.INTERNAL
    assert lib.nnb200_launch_count() == before
    torch.cuda.synchronize(dev)
    assert bool((out == 9).all()) and bool((other == 9).all())
    assert capi.take_device_error() == capi.DEVICE_ERROR_PEER_WAIT          # reading it clears the state
    capi.check(lib.nnb200_gemm_i8(C.byref(args), stream), "nnb200_gemm_i8")  # accepted again
    torch.cuda.synchronize(dev)
    assert bool((out[:, :256] == 0).all()) and bool((other[:, :256] == 0).all())
    assert capi.take_device_error() == 0


def test_rank_barrier_arguments_checked(nnb200_lib):
    from nnops_b200 import capi

    dev = torch.device("cuda:0")
    _, table = _flag_arrays(dev, 2)
    lib = capi.lib()
    for world, rank in ((0, 0), (9, 0), (2, 2), (2, -1)):
        assert lib.nnb200_rank_barrier(table, world, rank, 0, None) != capi.OK
    assert capi.take_device_error() == 0
