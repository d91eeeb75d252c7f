"""Column-sharded int8 Linear across the GPUs of one node.

Rank r owns output channels [r*N/g, (r+1)*N/g): the matching rows of W [N,K] (contiguous,
because W is row-major), and the matching slices of the per-channel scales and the bias.
Activations are replicated.  Each output element is produced by exactly one GPU from the same
integer inputs, so the g-way result is byte-identical to the single-GPU one.

Two ways to put the full row-major [M,N] output on every rank:

* ``mode="nccl"``  -- local GEMM into a dense [M, N/g] slab, NCCL all-gather over
  NVLink/NVSwitch into [g][M][N/g], then the library's interleave kernel writes [M,N].
* ``mode="multicast"`` -- like ``fused``, but the outputs are symmetric-memory allocations bound
  to one NVSwitch multicast object (``torch.distributed._symmetric_memory``: plumbing only), and
  the epilogue stores each tile ONCE with ``multimem.st``; the switch replicates it into every
  rank's copy.  A GPU then sends N/g columns instead of (g-1) times that.  Where the fabric
  offers no multicast the layer falls back to ``fused`` over the same allocations.
* ``mode="fused"`` -- the outputs are allocated with ``alloc_outputs`` (every rank maps every
  other rank's copy through CUDA IPC); the GEMM's epilogue then stores each finished tile into
  all g copies at once with peer-to-peer stores, so the all-gather overlaps the math tile by
  tile and no separate collective or re-layout pass runs.  Ranks are ordered after the GEMM
  (and optionally before it, when a consumer of the previous result may still be reading) by
  the library's device-side barrier -- every rank writes an epoch into every other rank's flag
  array and polls its own, with a bounded wait -- or, with ``rank_order="nccl"``, by a
  one-element all-reduce.  Kernels only ever LOAD local memory, except for that flag polling.

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


class RankLost(RuntimeError):
    """Another rank of the sharded layer has left, or has not been heard from in time."""

    def __init__(self, rank: int, why: str):
        self.rank, self.why = rank, why
        super().__init__(f"rank {rank} {why}")


class RankMonitor:
    """Host-side liveness of the ranks of a sharded layer, through a key-value store every rank
    can reach (``torch.distributed.TCPStore`` or any object with ``set`` / ``get`` / ``check``).

    The device-side barrier and the collectives assume every rank takes part; a rank that has
    died would leave the others waiting until a bounded wait runs out.  Before each step every
    rank therefore (1) publishes the step it is about to run and (2) waits until every other
    rank has published the same step: a rank that announced it is leaving instead (``leave``: a
    clean exit between steps) or that does not publish within ``timeout_s`` raises ``RankLost``
    on the host, BEFORE anything is launched, so no kernel or collective of the survivors is
    left in flight.  It costs a few store round trips per step, so it is opt-in.  The reference
    has no multi-GPU code; this sits above its operator API."""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 30.0, prefix: str = "nnb200"):
        self.store, self.rank, self.world, self.timeout_s, self.prefix = store, rank, world, float(timeout_s), prefix
        self.step = 0
        self.store.set(self._key("step", rank), "0")

    def _key(self, what: str, rank: int) -> str:
        return f"{self.prefix}/{what}/{rank}"

    def leave(self) -> None:
        """Tell the others this rank will run no further step (call between steps, nothing in flight)."""
        self.store.set(self._key("left", self.rank), "1")

    def begin_step(self) -> int:
        """Publish the next step and wait until every other rank has published it too.
        Returns the step number; raises RankLost otherwise."""
        import time
        self.step += 1
        self.store.set(self._key("step", self.rank), str(self.step))
        deadline = time.monotonic() + self.timeout_s
        for peer in range(self.world):
            if peer == self.rank:
                continue
            while True:
                seen = int(self.store.get(self._key("step", peer))) if self.store.check([self._key("step", peer)]) else -1
                if seen >= self.step:
                    break
                if self.store.check([self._key("left", peer)]):
                    raise RankLost(peer, "has left")
                if time.monotonic() > deadline:
                    raise RankLost(peer, f"has not reached step {self.step} within {self.timeout_s} s (last seen {seen})")
                time.sleep(0.002)
        return self.step


class _DeviceBuffer:
    """A library-allocated device buffer exposed to torch through __cuda_array_interface__."""

    def __init__(self, ptr: int, shape: tuple, kind: str):
        self.ptr = ptr
        self.__cuda_array_interface__ = {"shape": shape, "typestr": "|i1" if kind == "s8" else "|u1",
                                         "data": (ptr, False), "version": 2, "strides": None}

    def __del__(self):
        try:
            capi.lib().nnb200_peer_buffer_free(self.ptr)
        except Exception:
            pass


class ShardedLinearI8:
    """s8 x s8 Linear with the fused epilogue, N-sharded.  All tensors live on ``device``."""

    def __init__(self, w_shard: torch.Tensor, *, n_total: int, world: int, rank: int, group=None,
                 out_kind: str = "s8", bias_shard=None, scale_w_shard=1.0, scale_a=1.0, out_scale=1.0, out_zp=0,
                 relu: bool = False, mode: str = "nccl", rank_order: str = "device",
                 barrier_limit_cycles: int = 0):
        lo, hi = shard_bounds(n_total, world, rank)
        if w_shard.shape[0] != hi - lo:
            raise ValueError("weight shard has the wrong number of rows")
        if mode not in ("nccl", "fused", "multicast"):
            raise ValueError("mode must be 'nccl', 'fused' or 'multicast'")
        if mode in ("fused", "multicast") and out_kind not in ("s8", "u8"):
            raise ValueError("the fused write-back serves 8-bit outputs")
        self.w = w_shard
        self.n_total, self.world, self.rank, self.group = n_total, world, rank, group
        self.col0, self.n_per = lo, hi - lo
        self.out_kind = out_kind
        self.mode = mode if world > 1 else "nccl"
        self.kw = dict(bias=bias_shard, scale_w=scale_w_shard, scale_a=scale_a, out_scale=out_scale, out_zp=out_zp,
                       relu=relu)
        self._plans: dict = {}    # (a ptr, M, out ptr) -> prepared argument block + buffers
        self._last = None
        self._peer_ptrs: dict = {}    # local output data_ptr -> addresses of the other ranks' copies, mapped here
        self._mc_ptrs: dict = {}      # local output data_ptr -> address of the same buffer in the multicast mapping
        self.multicast_active = False
        self._owners: list = []
        self._token = None
        if rank_order not in ("device", "nccl"):
            raise ValueError("rank_order must be 'device' or 'nccl'")
        self.rank_order = rank_order     # how fused mode orders the ranks after the write-back
        # Wait limit of the device-side rank barrier in SM clock cycles; 0 = the library's default
        # (about half a minute: far longer than the pipeline waits inside a kernel, because ranks
        # drift apart by seconds for ordinary reasons).
        self.barrier_limit_cycles = int(barrier_limit_cycles)
        self._flags = None

    # ---- outputs -------------------------------------------------------------------------

    def alloc_outputs(self, m: int, count: int = 1) -> list[torch.Tensor]:
        """``count`` full [M, N] outputs on this rank.  In fused mode every rank must call this
        with the same arguments: the buffers are library allocations exported through CUDA IPC,
        and every rank maps every other rank's copies with ITS OWN device current (that is what
        makes them storable from its kernels)."""
        dev = self.w.device
        dt = ops._OUT_TORCH[self.out_kind]
        if self.mode == "nccl":
            return [torch.empty((m, self.n_total), dtype=dt, device=dev) for _ in range(count)]
        if self.mode == "multicast":
            return self._alloc_symmetric(m, count)
        lib = capi.lib()
        nbytes = m * self.n_total                    # 8-bit outputs
        outs, handles = [], []
        with torch.cuda.device(dev):
            for _ in range(count):
                ptr = C.c_void_p()
                capi.check(lib.nnb200_peer_buffer_alloc(C.byref(ptr), nbytes), "nnb200_peer_buffer_alloc")
                h = C.create_string_buffer(64)
                capi.check(lib.nnb200_peer_buffer_export(ptr, h), "nnb200_peer_buffer_export")
                owner = _DeviceBuffer(ptr.value, (m, self.n_total), self.out_kind)
                t = torch.as_tensor(owner, device=dev)
                self._owners.append(owner)
                outs.append(t)
                handles.append(h.raw)
            everyone: list = [None] * self.world
            dist.all_gather_object(everyone, handles, group=self.group)
            for i, t in enumerate(outs):
                mapped = []
                for r in range(self.world):
                    if r != self.rank:
                        p = C.c_void_p()
                        capi.check(lib.nnb200_peer_buffer_open(everyone[r][i], C.byref(p)), "nnb200_peer_buffer_open")
                        mapped.append(p.value)
                self._peer_ptrs[t.data_ptr()] = mapped
        self._token = torch.zeros(1, dtype=torch.int32, device=dev)
        if self.rank_order == "device" and self._flags is None:
            self._map_flags()
        dist.barrier(group=self.group)                   # every rank has mapped everything
        return outs

    def _alloc_symmetric(self, m: int, count: int) -> list[torch.Tensor]:
        """Outputs from torch's symmetric-memory allocator: every rank's buffer is mapped on every
        rank, and -- where the fabric supports it -- all of them are bound to one multicast
        object whose mapping ``multimem.st`` can store to."""
        import torch.distributed._symmetric_memory as symm_mem
        dev = self.w.device
        dt = ops._OUT_TORCH[self.out_kind]
        group = self.group if self.group is not None else dist.group.WORLD
        outs = []
        with torch.cuda.device(dev):
            for _ in range(count):
                t = symm_mem.empty((m, self.n_total), dtype=dt, device=dev)
                hdl = symm_mem.rendezvous(t, group)
                self._owners.append((t, hdl))
                mc = int(getattr(hdl, "multicast_ptr", 0) or 0)     # 0 where the fabric has no multicast
                if mc:
                    self._mc_ptrs[t.data_ptr()] = mc
                else:
                    self._peer_ptrs[t.data_ptr()] = [int(p) for r, p in enumerate(hdl.buffer_ptrs) if r != self.rank]
                outs.append(t)
        # Every rank must take the same path: multicast only if all of them have it.
        have = torch.tensor([1 if self._mc_ptrs else 0], dtype=torch.int32, device=dev)
        dist.all_reduce(have, op=dist.ReduceOp.MIN, group=self.group)
        self.multicast_active = bool(have.item())
        if not self.multicast_active and self._mc_ptrs:
            for (t, hdl) in [o for o in self._owners if isinstance(o, tuple)]:
                self._peer_ptrs[t.data_ptr()] = [int(p) for r, p in enumerate(hdl.buffer_ptrs) if r != self.rank]
            self._mc_ptrs.clear()
        self._token = torch.zeros(1, dtype=torch.int32, device=dev)
        if self.rank_order == "device" and self._flags is None:
            self._map_flags()
        dist.barrier(group=self.group)
        return outs

    def close(self) -> None:
        """Release the mapped and multicast-bound buffers while every rank is still alive: the
        ranks meet, each drops its allocations, and they meet again.  Call before the process
        group is destroyed."""
        if self.world > 1:
            torch.cuda.synchronize(self.w.device)
            dist.barrier(group=self.group)
        self._plans.clear()
        self._last = None
        self._peer_ptrs.clear()
        self._mc_ptrs.clear()
        self._owners.clear()
        self._flags = None
        if self.world > 1:
            torch.cuda.synchronize(self.w.device)
            dist.barrier(group=self.group)

    def _map_flags(self) -> None:
        """Flag arrays of the device-side rank barrier: one per rank, zeroed, mapped by every rank."""
        dev = self.w.device
        lib = capi.lib()
        ptr = C.c_void_p()
        capi.check(lib.nnb200_peer_buffer_alloc(C.byref(ptr), capi.RANK_FLAG_BYTES), "nnb200_peer_buffer_alloc")
        owner = _DeviceBuffer(ptr.value, (capi.RANK_FLAG_BYTES,), "u8")
        torch.as_tensor(owner, device=dev).zero_()
        torch.cuda.synchronize(dev)
        self._owners.append(owner)
        h = C.create_string_buffer(64)
        capi.check(lib.nnb200_peer_buffer_export(ptr, h), "nnb200_peer_buffer_export")
        everyone: list = [None] * self.world
        dist.all_gather_object(everyone, h.raw, group=self.group)
        table = (C.c_void_p * self.world)()
        for r in range(self.world):
            if r == self.rank:
                table[r] = ptr.value
            else:
                p = C.c_void_p()
                capi.check(lib.nnb200_peer_buffer_open(everyone[r], C.byref(p)), "nnb200_peer_buffer_open")
                table[r] = p.value
        self._flags = table

    def rank_barrier(self) -> None:
        """Order the ranks on the current stream: the library's device-side barrier (flags written
        into each other's memory) once ``alloc_outputs`` has mapped the flag arrays, else a
        one-element all-reduce."""
        if self.world <= 1:
            return
        if self._flags is not None:
            dev = self.w.device
            with torch.cuda.device(dev):
                capi.check(capi.lib().nnb200_rank_barrier(self._flags, self.world, self.rank, self.barrier_limit_cycles,
                                                          torch.cuda.current_stream(dev).cuda_stream),
                           "nnb200_rank_barrier")
            return
        if self._token is None:
            self._token = torch.zeros(1, dtype=torch.int32, device=self.w.device)
        dist.all_reduce(self._token, group=self.group)

    def check(self) -> None:
        """Synchronise this rank's device and raise if a bounded wait ran out since the last
        check: the outputs gathered since then are valid only if this passes.  (Without calling
        it, a barrier that timed out still makes the NEXT ``forward`` / ``rank_barrier`` on this
        rank fail with status ``internal`` -- the library keeps a sticky flag the host reads
        without synchronising.)"""
        with torch.cuda.device(self.w.device):
            code = capi.take_device_error()
        if code != 0:
            raise capi.Nnb200Error(capi.INTERNAL, f"device error word = {code}")

    # ---- compute -------------------------------------------------------------------------

    def _plan(self, a: torch.Tensor, out: torch.Tensor | None) -> dict:
        """Argument block and buffers for this (activations, destination) pair, built once."""
        m = a.shape[0]
        fused = self.mode in ("fused", "multicast") and out is not None and (
            out.data_ptr() in self._peer_ptrs or out.data_ptr() in self._mc_ptrs)
        direct = self.world == 1 or fused
        key = (a.data_ptr(), m, out.data_ptr() if (out is not None and direct) else 0)
        plan = self._plans.get(key)
        if plan is None:
            dt = ops._OUT_TORCH[self.out_kind]
            gathered = None
            if self.world == 1:
                # Single GPU: the GEMM writes the caller's output directly.
                slab = out if out is not None else torch.empty((m, self.n_per), dtype=dt, device=a.device)
            elif fused:
                slab = out[:, self.col0:self.col0 + self.n_per]        # this rank's window of its own copy
            else:
                slab = torch.empty((m, self.n_per), dtype=dt, device=a.device)
                gathered = torch.empty((self.world * m, self.n_per), dtype=dt, device=a.device)  # [g][M][N/g]
            keep: list = []
            args = ops.gemm_i8_args(a, self.w, slab, out_kind=self.out_kind, keep=keep, **self.kw)
            if fused and out.data_ptr() in self._mc_ptrs:
                args.multicast_out = self._mc_ptrs[out.data_ptr()] + self.col0 * out.element_size()
            elif fused:
                peers = self._peer_ptrs[out.data_ptr()]
                args.num_peer_outs = len(peers)
                for i, base in enumerate(peers):
                    args.peer_out[i] = base + self.col0 * out.element_size()   # same window, same pitch
            plan = dict(args=args, keep=keep, slab=slab, gathered=gathered, fused=fused)
            self._plans[key] = plan
        return plan

    def local(self, a: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """This rank's share of the work: the GEMM alone.  At g = 1 it writes ``out`` directly; in
        fused mode it writes this rank's column window of EVERY rank's ``out``."""
        plan = self._plan(a, out)
        with torch.cuda.device(a.device):
            capi.check(capi.lib().nnb200_gemm_i8(C.byref(plan["args"]),
                                                 torch.cuda.current_stream(a.device).cuda_stream), "nnb200_gemm_i8")
        self._last = plan
        return plan["slab"]

    def reassemble(self, out: torch.Tensor | None = None) -> torch.Tensor:
        """Make the full [M, N] of the last ``local`` call valid on this rank."""
        plan = self._last
        slab = plan["slab"]
        if self.world == 1:
            return slab
        if plan["fused"]:
            self.rank_barrier()       # every rank's tiles have landed in every copy
            return out
        m = slab.shape[0]
        if out is None:
            out = torch.empty((m, self.n_total), dtype=slab.dtype, device=slab.device)
        dist.all_gather_into_tensor(plan["gathered"], slab, group=self.group)
        esize = slab.element_size()
        with torch.cuda.device(slab.device):
            capi.check(capi.lib().nnb200_interleave_shards(
                plan["gathered"].data_ptr(), out.data_ptr(), m, self.n_per * esize, self.world, out.stride(0) * esize,
                torch.cuda.current_stream(slab.device).cuda_stream), "nnb200_interleave_shards")
        return out

    def forward(self, a: torch.Tensor, out: torch.Tensor | None = None, *, wait_for_readers: bool = False,
                monitor: "RankMonitor | None" = None) -> torch.Tensor:
        """Full row-major [M, N] output on every rank.  ``wait_for_readers``: in fused mode, order
        the ranks BEFORE the GEMM as well, for callers whose previous result in ``out`` may still
        be read on another rank when this call starts.  ``monitor``: check on the host that every
        rank is still there before anything is launched (raises RankLost)."""
        if monitor is not None and self.world > 1:
            monitor.begin_step()
        if wait_for_readers and self.mode in ("fused", "multicast"):
            self.rank_barrier()
        self.local(a, out)
        return self.reassemble(out)
