"""Column-sharded int8 Linear across the GPUs of one node.

Rank r owns output channels [r*N/g, (r+1)*N/g): the matching rows of W [N,K] (contiguous,
because W is row-major), and the matching slices of the per-channel scales and the bias.
Activations are replicated.  Each output element is produced by exactly one GPU from the same
integer inputs, so the g-way result is byte-identical to the single-GPU one.

Two ways to reassemble the [M,N] output on every rank:

* ``mode="nccl"``   -- local GEMM into a dense [M, N/g] slab, NCCL all-gather over
  NVLink/NVSwitch into [g][M][N/g], then the library's interleave kernel writes row-major [M,N].
* ``mode="fused"``  -- see ``PeerOutput`` (added by later steps of the build).

The reference has no multi-GPU code; this layer sits above its operator API, one operator
instance per GPU.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import capi, ops


def shard_bounds(n: int, world: int, rank: int) -> tuple[int, int]:
    """Half-open channel range of ``rank``.  N must divide evenly so that every rank gathers
    equally sized slabs."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad world/rank")
    if n % world:
        raise ValueError(f"N={n} is not divisible by {world} ranks")
    per = n // world
    return rank * per, (rank + 1) * per


def shard_rows(t, world: int, rank: int):
    """Slice a per-channel array or the [N,K] weight along its first dimension."""
    lo, hi = shard_bounds(t.shape[0], world, rank)
    return t[lo:hi]


class ShardedLinearI8:
    """s8 x s8 Linear with the fused epilogue, N-sharded.  All tensors live on ``device``."""

    def __init__(self, w_shard: torch.Tensor, *, n_total: int, world: int, rank: int, group=None,
                 out_kind: str = "s8", bias_shard=None, scale_w_shard=1.0, scale_a=1.0, out_scale=1.0, out_zp=0,
                 relu: bool = False):
        lo, hi = shard_bounds(n_total, world, rank)
        if w_shard.shape[0] != hi - lo:
            raise ValueError("weight shard has the wrong number of rows")
        self.w = w_shard
        self.n_total, self.world, self.rank, self.group = n_total, world, rank, group
        self.n_per = hi - lo
        self.out_kind = out_kind
        self.kw = dict(bias=bias_shard, scale_w=scale_w_shard, scale_a=scale_a, out_scale=out_scale, out_zp=out_zp,
                       relu=relu)
        self._plans: dict = {}   # (a ptr, M, out ptr) -> prepared argument block + buffers
        self._last = None

    def _plan(self, a: torch.Tensor, out: torch.Tensor | None) -> dict:
        """Argument block and buffers for this (activations, destination) pair, built once."""
        m = a.shape[0]
        key = (a.data_ptr(), m, out.data_ptr() if (out is not None and self.world == 1) else 0)
        plan = self._plans.get(key)
        if plan is None:
            dt = ops._OUT_TORCH[self.out_kind]
            if self.world == 1:
                # Single GPU: the GEMM writes the caller's output directly.
                slab = out if out is not None else torch.empty((m, self.n_per), dtype=dt, device=a.device)
                gathered = None
            else:
                slab = torch.empty((m, self.n_per), dtype=dt, device=a.device)
                gathered = torch.empty((self.world * m, self.n_per), dtype=dt, device=a.device)  # [g][M][N/g]
            keep: list = []
            args = ops.gemm_i8_args(a, self.w, slab, out_kind=self.out_kind, keep=keep, **self.kw)
            plan = dict(args=args, keep=keep, slab=slab, gathered=gathered)
            self._plans[key] = plan
        return plan

    def local(self, a: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """This rank's [M, N/g] slab: the GEMM alone (written straight into ``out`` at g = 1)."""
        plan = self._plan(a, out)
        capi.check(capi.lib().nnb200_gemm_i8(C.byref(plan["args"]), torch.cuda.current_stream(a.device).cuda_stream),
                   "nnb200_gemm_i8")
        self._last = plan
        return plan["slab"]

    def reassemble(self, out: torch.Tensor | None = None) -> torch.Tensor:
        """All-gather the slabs of the last ``local`` call and interleave them into [M, N]."""
        plan = self._last
        slab = plan["slab"]
        if self.world == 1:
            return slab
        m = slab.shape[0]
        if out is None:
            out = torch.empty((m, self.n_total), dtype=slab.dtype, device=slab.device)
        dist.all_gather_into_tensor(plan["gathered"], slab, group=self.group)
        esize = slab.element_size()
        capi.check(capi.lib().nnb200_interleave_shards(
            plan["gathered"].data_ptr(), out.data_ptr(), m, self.n_per * esize, self.world, out.stride(0) * esize,
            torch.cuda.current_stream(slab.device).cuda_stream), "nnb200_interleave_shards")
        return out

    def forward(self, a: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """Full row-major [M, N] output on every rank."""
        self.local(a, out)
        return self.reassemble(out)
