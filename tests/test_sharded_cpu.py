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
