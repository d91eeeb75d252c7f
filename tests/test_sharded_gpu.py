"""Column-sharded int8 Linear on real GPUs: g ranks over NCCL must reproduce the single-GPU
output byte for byte (and that one equals the oracle).  Needs at least two GPUs; skipped
otherwise."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, m: int, n: int, k: int, mode: str, q):
    import torch.distributed as dist
    from nnops_b200 import capi, synth
    from nnops_b200.sharded import ShardedLinearI8, shard_rows
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        _rank_body(rank, world, m, n, k, mode, q, dev)
    except Exception:  # report instead of leaving the parent to time out
        import traceback
        q.put((rank, "ERROR: " + traceback.format_exc()))
    finally:
        dist.destroy_process_group()


def _rank_body(rank, world, m, n, k, mode, q, dev):
    import torch.distributed as dist
    from nnops_b200 import capi, synth
    from nnops_b200.sharded import ShardedLinearI8, shard_rows
    c = synth.config2(m=m, n=n, k=k, out_scale=1.6)
    layer = ShardedLinearI8(
        torch.from_numpy(np.ascontiguousarray(shard_rows(c.w, world, rank))).to(dev), n_total=n, world=world,
        rank=rank, out_kind="s8", relu=True, scale_a=c.scale_a, out_scale=c.out_scale,
        bias_shard=torch.from_numpy(np.ascontiguousarray(shard_rows(c.bias, world, rank))).to(dev),
        scale_w_shard=torch.from_numpy(np.ascontiguousarray(shard_rows(c.scale_w, world, rank))).to(dev),
        mode="fused" if mode.startswith("fused") else mode,
        rank_order="nccl" if mode == "fused-nccl-order" else "device")
    a = torch.from_numpy(c.a).to(dev)
    if mode.startswith("fused") or mode == "multicast":
        # From here to layer.close() no rank may leave early: the buffers are mapped (and, with
        # multicast, bound to one switch object) on every rank, so problems are recorded and
        # raised only after all ranks have released them together.
        problem = None
        outs = layer.alloc_outputs(m, count=2)                           # peer-mapped on every rank
        for o in outs:
            o.fill_(0x5A)
        torch.cuda.synchronize()
        dist.barrier()
        for i in range(12):                                              # alternate buffers, reuse them
            if rank == i % world:
                torch.cuda._sleep(2_000_000)                             # a different straggler every round
            layer.forward(a, outs[i & 1], wait_for_readers=True)
        torch.cuda.synchronize()
        if not torch.equal(outs[0], outs[1]):
            problem = "the two output buffers differ"
        result = torch.full((m, n + 32), 0x5A, dtype=torch.int8, device=dev)
        result[:, :n] = outs[1]
        if mode == "multicast" and rank == 0:
            print(f"multicast stores active: {layer.multicast_active}")
        err = capi.take_device_error()
        if err != 0:
            problem = f"device error word {err}"
        del outs
        layer.close()
        if problem is not None:
            raise AssertionError(problem)
    else:
        result = torch.full((m, n + 32), 0x5A, dtype=torch.int8, device=dev)   # pitched destination
        for _ in range(2):                                                      # twice: buffers are reused
            layer.forward(a, result[:, :n])
    torch.cuda.synchronize()
    assert capi.take_device_error() == 0
    dist.barrier()
    q.put((rank, result.cpu().numpy()))


@pytest.mark.parametrize("mode", ["nccl", "fused", "fused-nccl-order", "multicast"])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_matches_single_gpu(nnb200_lib, world, mode):
    _run_sharded(world, mode, 512, 2048, 1024)


@pytest.mark.parametrize("world", [2, 8])
def test_sharded_multicast_wide_shard(nnb200_lib, world):
    """A shard of 3584 channels with 4096 rows: the width at which the multicast form takes
    224-column tiles (ragged against the 128-column staging groups)."""
    _run_sharded(world, "multicast", 4096, 3584 * world, 256, check_oracle=False)


def _run_sharded(world, mode, m, n, k, check_oracle=True):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    import oracle
    from nnops_b200 import ops, synth
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, m, n, k, mode, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=240) for _ in range(world))
    for p in procs:
        p.join(timeout=240)
    for r, v in results.items():
        assert not isinstance(v, str), f"rank {r}: {v}"
    for p in procs:
        assert p.exitcode == 0
    c = synth.config2(m=m, n=n, k=k, out_scale=1.6)
    dev = torch.device("cuda:0")
    single = ops.gemm_i8(torch.from_numpy(c.a).to(dev), torch.from_numpy(c.w).to(dev), **c.kwargs()).cpu().numpy()
    if check_oracle:
        assert np.array_equal(single, oracle.gemm_i8(c.a, c.w, **c.kwargs()))
    for r in range(world):
        assert np.array_equal(results[r][:, :n], single), f"rank {r} differs from the single-GPU result"
        assert np.all(results[r][:, n:] == 0x5A), "padding of the pitched output was touched"
