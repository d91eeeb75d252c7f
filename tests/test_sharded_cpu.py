"""Host-side logic of the column-sharded Linear, on CPU ranks: shard arithmetic, the layout an
all-gather produces, and its reassembly into the row-major output.  Two gloo ranks stand in for
two GPUs; each rank's slab comes from the CPU oracle (this is a test of the plumbing, not of
the kernels), and the reassembled result must equal the unsharded oracle result byte for byte.
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from nnops_b200 import synth
from nnops_b200.sharded import shard_bounds, shard_rows


def test_shard_bounds():
    assert shard_bounds(28672, 8, 0) == (0, 3584)
    assert shard_bounds(28672, 8, 7) == (25088, 28672)
    assert [shard_bounds(12, 4, r) for r in range(4)] == [(0, 3), (3, 6), (6, 9), (9, 12)]
    with pytest.raises(ValueError):
        shard_bounds(10, 4, 0)      # uneven shards cannot be all-gathered
    with pytest.raises(ValueError):
        shard_bounds(8, 2, 2)


def test_shards_tile_the_weight():
    w = np.arange(24).reshape(12, 2)
    parts = [shard_rows(w, 3, r) for r in range(3)]
    assert np.array_equal(np.concatenate(parts), w)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, m: int, n: int, k: int, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        c = synth.config2(m=m, n=n, k=k, out_scale=1.6)
        kw = c.kwargs()
        kw["bias"] = shard_rows(c.bias, world, rank)
        kw["scale_w"] = shard_rows(c.scale_w, world, rank)
        slab = torch.from_numpy(oracle.gemm_i8(c.a, np.ascontiguousarray(shard_rows(c.w, world, rank)), **kw))
        gathered = torch.empty((world * m, n // world), dtype=slab.dtype)   # rank-major concatenation
        dist.all_gather_into_tensor(gathered, slab)
        # What nnb200_interleave_shards does on the device: [g][M][N/g] -> [M][g*N/g].
        full = gathered.view(world, m, n // world).permute(1, 0, 2).reshape(m, n).contiguous()
        q.put((rank, full.numpy()))
    finally:
        dist.destroy_process_group()


def test_two_rank_gather_matches_unsharded():
    m, n, k = 48, 64, 96
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, m, n, k, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    c = synth.config2(m=m, n=n, k=k, out_scale=1.6)
    want = oracle.gemm_i8(c.a, c.w, **c.kwargs())
    for r in range(world):
        assert np.array_equal(results[r], want)


# ---- host-side failure detection: a rank that leaves, a rank that stalls ---------------------------
# The failures are made on the host (a rank that announces its exit between steps; a rank that
# stops publishing), with gloo ranks on CPU; nothing here touches a GPU.

def _monitor_rank(rank: int, world: int, port: int, store_port: int, scenario: str, q):
    from nnops_b200.sharded import RankLost, RankMonitor
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    store = dist.TCPStore("127.0.0.1", store_port, world, rank == 0, wait_for_workers=True)
    mon = RankMonitor(store, rank, world, timeout_s=1.0)
    token = torch.zeros(1)
    steps_done, lost = 0, None
    try:
        for step in range(1, 6):
            if scenario == "leaves" and rank == 1 and step == 3:
                mon.leave()                      # between steps, nothing in flight
                break
            if scenario == "stalls" and rank == 1 and step == 3:
                import time
                time.sleep(3.0)                  # never publishes step 3 in time
                break
            try:
                mon.begin_step()
            except RankLost as e:
                lost = (e.rank, e.why)
                break
            dist.all_reduce(token)               # stands for the step's collective / device barrier
            steps_done += 1
    finally:
        q.put((rank, steps_done, lost))
        if scenario == "stalls" and rank != 1:
            import time
            time.sleep(2.5)                      # let the stalled rank finish before the store owner exits
        dist.destroy_process_group()


@pytest.mark.parametrize("scenario", ["leaves", "stalls"])
def test_lost_rank_is_reported_on_the_host_before_the_next_step(scenario):
    world = 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port, store_port = _free_port(), _free_port()
    procs = [ctx.Process(target=_monitor_rank, args=(r, world, port, store_port, scenario, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = {r: (done, lost) for r, done, lost in (q.get(timeout=120) for _ in range(world))}
    for p in procs:
        p.join(timeout=60)
    # Rank 1 ran two whole steps.  The others completed exactly those two, then learnt on the
    # host -- before launching step 3 -- that rank 1 was gone; no collective was left hanging.
    assert results[1][0] == 2
    for r in (0, 2):
        done, lost = results[r]
        assert done == 2, results
        assert lost is not None and lost[0] == 1, results
        assert ("left" in lost[1]) if scenario == "leaves" else ("not reached" in lost[1])
