#!/usr/bin/env python
"""Benchmark of the quantized-matmul hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (all N): the sharded int8 QuantLinear configuration -- A s8 [4096,8192] x W s8
[28672,8192] -> s8 [4096,28672] with int32 bias, Relu and per-channel requantisation -- on
seeded synthetic tensors.  At N > 1 W, scales and bias are column-sharded N/g per rank and the
[M,N] output is reassembled on every rank (NCCL all-gather + interleave); total work is fixed,
so scaling is "strong".  One step = one pass of that path.  Prints ONE JSON line (rank 0).

``--impl reference`` times the reference's own CPU implementation of the same path
(oracle/_ref when it was compiled, else the C restatement) on the host cores, on the same
whole configuration.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

M, N, K = 4096, 28672, 8192
METRIC = "int8_quantlinear_tops"
UNIT = "TOPS"
WORKLOAD = "sharded int8 QuantLinear s8[4096,8192] x s8[28672,8192] -> s8, bias+Relu+per-channel requant"


def read_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class NvmlSampler:
    """SM clock and clock-event reasons read through NVML from a thread of this process, every
    couple of milliseconds, while the timed region runs (read-only queries)."""

    def __init__(self, gpu_index: int, uuid: str | None = None):
        import threading
        import pynvml
        self.nv = pynvml
        pynvml.nvmlInit()
        handle = None
        if uuid:
            try:
                handle = pynvml.nvmlDeviceGetHandleByUUID(uuid if uuid.startswith("GPU-") else "GPU-" + uuid)
            except pynvml.NVMLError:
                handle = None
        self.h = handle if handle is not None else pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
        self.sm, self.mask, self.power = [], 0, []
        self.smax = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                self.mask |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                self.power.append(nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0)
            except nv.NVMLError:
                pass
            time.sleep(0.002)

    def start(self):
        self._thread.start()

    def stop(self) -> dict:
        self._stop.set()
        self._thread.join(timeout=2)
        nv = self.nv
        names = (("hw_slowdown", nv.nvmlClocksEventReasonHwSlowdown),
                 ("hw_thermal_slowdown", nv.nvmlClocksEventReasonHwThermalSlowdown),
                 ("sw_thermal_slowdown", nv.nvmlClocksEventReasonSwThermalSlowdown),
                 ("sw_power_cap", nv.nvmlClocksEventReasonSwPowerCap))
        reasons = sorted(n for n, bit in names if self.mask & bit)
        return {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": float(self.smax),
                "samples": len(self.sm), "reasons": reasons, "source": "nvml, 2 ms period, timed region only",
                "power_w": round(statistics.median(self.power), 1) if self.power else None}


def make_clock_sampler(gpu_index: int, uuid: str | None = None):
    """(sampler, tight): the in-process NVML sampler when NVML is usable -- it brackets the timed
    region tightly -- else the nvidia-smi subprocess, which needs slack before and after."""
    try:
        return NvmlSampler(gpu_index, uuid), True
    except Exception:
        return ClockSampler(gpu_index), False


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, smax, reasons = [], [], set()
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # Under load = the upper half of the samples (idle samples before/after are excluded).
        load = sorted(sm)[len(sm) // 2:] if sm else []
        return {"sm_mhz": statistics.median(load) if load else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def host_cores() -> dict:
    """Logical CPUs this process may use, and the physical cores / SMT width behind them as
    /proc/cpuinfo describes them (None where it does not say)."""
    logical = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    cores, siblings, per_pkg = set(), None, None
    try:
        phys = core = None
        with open("/proc/cpuinfo") as f:
            for line in f:
                key, _, val = line.partition(":")
                key, val = key.strip(), val.strip()
                if key == "physical id":
                    phys = val
                elif key == "core id":
                    core = val
                elif key == "siblings":
                    siblings = int(val)
                elif key == "cpu cores":
                    per_pkg = int(val)
                elif key == "" and phys is not None and core is not None:
                    cores.add((phys, core))
                    phys = core = None
    except (OSError, ValueError):
        pass
    smt = (siblings // per_pkg) if siblings and per_pkg else None
    physical = len(cores) if cores else None
    if physical and smt and physical * smt < logical:
        physical = None      # a container that hides part of the topology: do not guess
    return {"logical": logical, "physical": physical, "smt": smt}


def cpu_reference_run(rows: int, steps: int, warmup: int, keep_output: bool = False):
    """Reference CPU route (or the C restatement when it is not runnable here) on the first
    ``rows`` rows of A against all of W, with all the host threads it can use."""
    import oracle
    from nnops_b200 import synth
    c = synth.config5()
    a = c.a if rows >= M else np.ascontiguousarray(c.a[:rows])
    use_ref = oracle.have_ref()
    hc = host_cores()
    threads = hc["logical"]
    kw = c.kwargs()

    def call():
        if use_ref:
            return oracle.gemm_i8(a, c.w, impl="ref", threads=threads, **kw)
        return oracle.gemm_i8(a, c.w, impl="port", **kw)

    out = None
    for _ in range(warmup):
        out = call()
    t0 = time.perf_counter()
    for _ in range(steps):
        out = call()
    dt = (time.perf_counter() - t0) / steps
    ops_count = 2.0 * a.shape[0] * N * K
    what = f"all {M} activation rows" if a.shape[0] >= M else f"first {a.shape[0]} of {M} activation rows"
    r = {"value": ops_count / dt / 1e12, "unit": UNIT, "cores": threads if use_ref else 1,
         "physical_cores": hc["physical"], "smt": hc["smt"],
         "kind": "reference" if use_ref else "port",
         "sample": f"{what} x all {N} channels, K={K}; {steps} timed calls after {warmup} warm-ups, wall clock",
         "ms_per_call": dt * 1e3, "rows": int(a.shape[0])}
    if keep_output:
        r["output"] = out
    return r


def cpu_q4_1_baseline() -> dict:
    """The Q4_1 half of the metric on the host: the reference's Linear(f32 x q4_1, Backend::CPU)
    on the decode-step configuration (M = 1 and 8, K = N = 4096), in GB/s of the same algorithmic
    bytes the GPU figure counts, with all host threads and with one.  Method of the reference's
    operator bench (tests/bench_linear.cpp:127-163): 3 warm-ups, then rounds of at least 8 calls
    and 100 ms; the median of 3 rounds."""
    import oracle
    from nnops_b200 import synth
    hc = host_cores()
    if not oracle.have_ref():
        return {"unavailable": "compiled reference route not runnable on this host"}
    out = {"unit": "GB/s", "kind": "reference", "cores": hc["logical"], "physical_cores": hc["physical"],
           "smt": hc["smt"],
           "method": "Linear(f32 x q4_1, Backend::CPU), f32 activations holding the f16 values; 3 warm-ups, "
                     "median of 3 rounds of >= 8 calls and >= 100 ms; bytes = the GPU figure's algorithmic bytes"}
    for m in (1, 8):
        c = synth.config3(m)
        a32 = c.a.astype(np.float32)
        for label, threads in (("all_cores", hc["logical"]), ("one_thread", 1)):
            def call():
                oracle.q4_1_matmul(a32, c.w_blocks, c.k, out_dtype="f32", impl="ref", threads=threads)
            for _ in range(3):
                call()
            rounds = []
            for _ in range(3):
                n_calls, t0 = 0, time.perf_counter()
                while n_calls < 8 or time.perf_counter() - t0 < 0.1:
                    call()
                    n_calls += 1
                rounds.append((time.perf_counter() - t0) / n_calls)
            out[f"m{m}_{label}"] = c.bytes / statistics.median(rounds) / 1e9
    return out


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # The whole configuration, every step: one call is well under two seconds of CPU time.
    r = cpu_reference_run(M, max(1, args.steps), max(1, args.warmup))
    line = {
        "impl": "reference", "metric": METRIC, "value": r["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_call"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "s8", "data": "synthetic",
        "config": {"workload": WORKLOAD, "m": M, "n": N, "k": K},
        "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "physical_cores", "smt", "kind", "sample")},
        "e2e": {"value": r["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def secondary_q4_1(torch, dev, peaks, gemv_only: bool = False):
    """Q4_1 decode GEMV (M=1, M=8) in HBM GB/s and the prefill GEMM in TFLOP/s, reported beside
    the headline.  The 10 MiB weight matrix fits in L2, so the GEMV cycles over enough distinct
    weight replicas (>= 3x L2) inside one CUDA graph that every launch streams from HBM."""
    from nnops_b200 import ops, synth
    out = {}
    l2 = torch.cuda.get_device_properties(dev).L2_cache_size
    for m in (1, 8):
        c = synth.config3(m)
        reps = max(8, int(3 * l2 // c.w_blocks.size) + 1)
        w0 = torch.from_numpy(c.w_blocks).to(dev)
        ws = [w0] + [w0.clone() for _ in range(reps - 1)]
        a = torch.from_numpy(c.a).to(dev)
        o = torch.empty((m, c.w_blocks.shape[0]), dtype=torch.float32, device=dev)
        for w in ws[:3]:
            ops.linear_q4_1(a, w, c.k, out=o)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            with torch.cuda.graph(g, stream=s):
                for w in ws:
                    # Back-to-back decode GEMVs: each launch may start fetching its weights while
                    # the previous one drains (programmatic dependent launch).
                    ops.linear_q4_1(a, w, c.k, out=o, overlap_previous=True)
        torch.cuda.synchronize()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        iters = 20
        e0.record()
        for _ in range(iters):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (iters * reps)
        gbs = c.bytes / us / 1e3
        out[f"q4_1_gemv_m{m}"] = {"gbs": gbs, "us_per_call": us, "bytes_per_call": c.bytes,
                                  "frac_of_hbm_peak": gbs / peaks["hbm_gbs"], "replicas": reps,
                                  "method": "CUDA graph of one launch per weight replica (replicas >= 3x L2), "
                                            "launches chained with programmatic dependent launch"}
        del ws, g
    if gemv_only:
        return out
    c = synth.config4()
    a, w = torch.from_numpy(c.a).to(dev), torch.from_numpy(c.w_blocks).to(dev)
    o = torch.empty((c.a.shape[0], c.w_blocks.shape[0]), dtype=torch.float16, device=dev)
    # The whole call (auto picks the two-pass form here: expansion of W + dense GEMM), and the
    # fused single-kernel form beside it.
    for key, engine in (("q4_1_gemm", "auto"), ("q4_1_gemm_fused", "gemm")):
        for _ in range(3):
            ops.linear_q4_1(a, w, c.k, out=o, engine=engine)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            ops.linear_q4_1(a, w, c.k, out=o, engine=engine)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / 10
        tf = c.flops / ms / 1e9
        out[key] = {"tflops": tf, "ms_per_call": ms, "frac_of_bf16_peak": tf / peaks["bf16_tflops"],
                    "engine": ops.q4_1_engine(a, w, c.k, out_dtype=torch.float16, engine=engine)}
    return out


def graph_time_us(torch, fn, calls_per_graph: int = 10, replays: int = 10) -> float:
    """Average device time of one ``fn()`` call: ``calls_per_graph`` calls captured in a CUDA
    graph (so host-side launch cost does not pace the kernels), replayed between two events."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            for _ in range(calls_per_graph):
                fn()
    torch.cuda.synchronize()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (replays * calls_per_graph)


def secondary_i8_decode(torch, dev, peaks, w, sw, bias):
    """The int8 layer's token-by-token twin: M = 1, 8, 16 activation rows against the bench's
    own weight matrix (235 MB, larger than L2, so every call streams it from HBM)."""
    from nnops_b200 import ops
    out = {}
    n, k = w.shape
    for m in (1, 8, 16):
        a = torch.randint(-127, 128, (m, k), dtype=torch.int8, device=dev)
        o = torch.empty((m, n), dtype=torch.int8, device=dev)
        kw = dict(out_kind="s8", out=o, bias=bias, relu=True, scale_a=0.02, scale_w=sw, out_scale=0.05)
        engine = ops.gemm_i8_engine(a, w, o, **{x: y for x, y in kw.items() if x != "out"})
        us = graph_time_us(torch, lambda: ops.gemm_i8(a, w, **kw))
        nbytes = n * k + m * k + m * n + 8 * n
        gbs = nbytes / us / 1e3
        out[f"i8_decode_m{m}"] = {"gbs": gbs, "us_per_call": us, "bytes_per_call": nbytes, "engine": engine,
                                  "frac_of_hbm_peak": gbs / peaks["hbm_gbs"]}
    return out


def secondary_quant_linear(torch, dev, peaks):
    """The elementwise steps either side of the int8 layer, on the bench's own tensors:
    QuantizeLinear of the [4096, 8192] activations (per token; f32 and f16 sources) and
    DequantizeLinear of the [4096, 28672] result (per tensor, to f16).  Pure streaming: bytes
    read + written over time, against the measured copy bandwidth.  All tensors exceed L2."""
    from nnops_b200 import ops
    out = {}

    def timed(fn, nbytes, key):
        us = graph_time_us(torch, fn)
        out[key] = {"gbs": nbytes / us / 1e3, "us_per_call": us, "bytes_per_call": nbytes,
                    "frac_of_hbm_peak": nbytes / us / 1e3 / peaks["hbm_gbs"]}

    scale = torch.full((M,), 0.02, dtype=torch.float32, device=dev)
    zp = torch.zeros(M, dtype=torch.int8, device=dev)
    for name, dt, esz in (("f32", torch.float32, 4), ("f16", torch.float16, 2)):
        x = torch.randn((M, K), dtype=dt, device=dev)
        q = torch.empty((M, K), dtype=torch.int8, device=dev)
        timed(lambda: ops.quantize_linear(x, scale, zp, out=q), M * K * (esz + 1), f"quantize_{name}_per_token")
        del x
    y = torch.randint(-128, 128, (M, N), dtype=torch.int8, device=dev)
    f = torch.empty((M, N), dtype=torch.float16, device=dev)
    s1 = torch.tensor([0.05], dtype=torch.float32, device=dev)
    z1 = torch.zeros(1, dtype=torch.int8, device=dev)
    timed(lambda: ops.dequantize_linear(y, s1, z1, out=f), M * N * 3, "dequantize_s8_to_f16_per_tensor")
    return out


def secondary_i8_config2(torch, dev, peaks):
    """The Llama-7B MLP shape of the benchmark's second configuration (M=512, N=11008, K=4096,
    s8 out, per-channel requant, ReLU), cycling over enough weight copies to exceed L2."""
    from nnops_b200 import ops, synth
    c = synth.config2()
    a = torch.from_numpy(c.a).to(dev)
    w0 = torch.from_numpy(c.w).to(dev)
    ws = [w0] + [w0.clone() for _ in range(5)]
    o = torch.empty((c.a.shape[0], c.w.shape[0]), dtype=torch.int8, device=dev)
    kw = {k: (torch.from_numpy(v).to(dev) if isinstance(v, np.ndarray) else v) for k, v in c.kwargs().items()}
    kw.pop("out_kind", None)

    def fn():
        for w in ws:
            ops.gemm_i8(a, w, out_kind="s8", out=o, **kw)

    us = graph_time_us(torch, fn, calls_per_graph=2) / len(ws)
    ops_count = 2.0 * c.a.shape[0] * c.w.shape[0] * c.a.shape[1]
    tops = ops_count / us / 1e6
    return {"i8_config2": {"tops": tops, "us_per_call": us, "frac_of_int8_peak": tops / (2.0 * peaks["bf16_tflops"])}}


def measured_i8_peak(torch, lib, dev, sampler_factory):
    """The part's int8 tensor rate from the library's issue-bound probe (tcgen05.mma kind::i8 on
    shared-memory-resident tiles).  Zero operands give the pipe's issue rate (best of five short
    launches); pseudo-random operands, in a loop of about two seconds with the SM clock sampled
    inside it, give what the same instruction stream holds under the power cap."""
    stream = torch.cuda.current_stream(dev).cuda_stream
    ops = C.c_double(0.0)

    def one(iters, pattern):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        st = lib.nnb200_measure_i8_mma_peak(iters, pattern, C.byref(ops), stream)
        e1.record()
        if st != 0:
            raise RuntimeError(f"nnb200_measure_i8_mma_peak: status {st}")
        torch.cuda.synchronize()
        return ops.value / (e0.elapsed_time(e1) * 1e-3) / 1e12

    def loop(pattern, launches, iters):
        sampler = sampler_factory()
        if sampler is not None:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(launches):
            lib.nnb200_measure_i8_mma_peak(iters, pattern, C.byref(ops), stream)
        e1.record()
        torch.cuda.synchronize()
        clocks = sampler.stop() if sampler is not None else None
        secs = e0.elapsed_time(e1) * 1e-3
        return {"tops": ops.value * launches / secs / 1e12, "seconds": secs, "clocks": clocks}

    # The half-second zero-operand loop first: it also brings the SM clock up, which short
    # launches after a memory-bound or idle stretch do not (a burst probe run cold read 3686
    # instead of 4565 TOP/s on the same GPU).
    sustained_zero = loop(0, 8, 1 << 18)
    one(2048, 0)
    burst = max(one(8192, 0) for _ in range(5))
    burst_random = max(one(8192, 1) for _ in range(5))
    return {"burst_tops": burst, "burst_tops_random_operands": burst_random,
            "sustained_zero_operands": sustained_zero, "sustained_random_operands": loop(1, 24, 1 << 18),
            "method": "one CTA per SM issuing tcgen05.mma.kind::i8 M128xN256xK32 back to back on shared-memory "
                      "tiles (zeros / pseudo-random bytes), two alternating TMEM accumulators; no loads, no epilogue"}


def sustained_gemm(torch, layer, a, out, total_ops, sampler_factory, seconds: float = 2.5):
    """The headline GEMM back to back for a couple of seconds: what it holds under the power cap."""
    for _ in range(3):
        layer.local(a, out)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = sampler_factory()
    if sampler is not None:
        sampler.start()
    launches = 0
    t_end = time.perf_counter() + seconds
    e0.record()
    while time.perf_counter() < t_end:
        # Chunks of 200 launches (~0.1 s) with one synchronisation each, so that the host clock
        # that ends the loop and the device stay together; the gap per chunk is microseconds.
        for _ in range(200):
            layer.local(a, out)
        launches += 200
        torch.cuda.synchronize()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop() if sampler is not None else None
    secs = e0.elapsed_time(e1) * 1e-3
    tops = total_ops * launches / secs / 1e12
    r = {"tops": tops, "seconds": secs, "launches": launches, "clocks": clocks}
    if clocks and clocks.get("sm_mhz") and clocks.get("sm_max_mhz"):
        r["tops_at_max_clock"] = tops * clocks["sm_max_mhz"] / clocks["sm_mhz"]
    return r


def operator_level_bench(steps: int, warmup: int):
    """The same layer driven from C++ through Linear::create(attrs, Backend::CUDA)->compute() with
    the weight scales as HOST arrays (tests/cpp/bench_linear_op.cpp): the drop-in build when it
    exists, else the stand-alone front end."""
    bin_dir = ROOT / "tests" / "cpp" / "_bin"
    for name in ("bench_linear_op_dropin", "bench_linear_op_standalone"):
        exe = bin_dir / name
        if exe.exists():
            try:
                r = subprocess.run([str(exe), str(M), str(N), str(K), str(steps), str(warmup)], capture_output=True,
                                   text=True, timeout=300)
                line = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
                if r.returncode == 0 and line:
                    d = json.loads(line[-1])
                    d["binary"] = name
                    return d
                return {"unavailable": f"{name} exited {r.returncode}: {(r.stdout + r.stderr)[-200:]}"}
            except (OSError, subprocess.TimeoutExpired, ValueError) as e:
                return {"unavailable": f"{name}: {e}"}
    return {"unavailable": "tests/cpp/_bin/bench_linear_op_* not built (python -m nnops_b200.host.build)"}


def secondary_i8_poses(torch, dev):
    """MatMul's four operand poses at 4096^3, s8 x s8 -> s32 (the reference quotes its own tile
    kernel on this shape, src/backend/cuda/matmul/matmul_i8_ptx.cu:474-479): 'nn' is MatMul's
    default, A [M, K] x B [K, N]; 'nt' is Linear's pose."""
    from nnops_b200 import ops
    size = 4096
    out = {}
    o = torch.empty((size, size), dtype=torch.int32, device=dev)
    for pose in ("nt", "nn", "tn", "tt"):
        a_store = torch.randint(-127, 128, (size, size), dtype=torch.int8, device=dev)
        b_store = torch.randint(-127, 128, (size, size), dtype=torch.int8, device=dev)
        a = a_store.t() if pose[0] == "t" else a_store
        w = b_store if pose[1] == "t" else b_store.t()
        engine = ops.gemm_i8_engine(a, w, o, out_kind="s32")
        us = graph_time_us(torch, lambda: ops.gemm_i8(a, w, out_kind="s32", out=o))
        out[f"i8_matmul_{pose}_4096"] = {"tops": 2.0 * size ** 3 / us / 1e6, "us_per_call": us, "engine": engine}
    return out


def secondary_i8_epilogue_bound(torch, dev, peaks):
    """Two int8 Linear calls whose time is the epilogue's, not the main loop's: a short K with an s8
    destination (the GEMM of a 1x1 convolution: M = 100352, N = 1024, K = 256, bias + ReLU +
    per-channel requant), and f16 / f32 destinations (dequantising epilogue with an f16 bias) at
    M = 32768, N = 4096, K = 256; and the headline-sized 8192^3 into f16.  Synthetic values."""
    from nnops_b200 import ops
    out = {}

    def case(key, m, n, k, kind, **kw):
        a = torch.randint(-127, 128, (m, k), dtype=torch.int8, device=dev)
        w = torch.randint(-127, 128, (n, k), dtype=torch.int8, device=dev)
        sw = torch.rand(n, device=dev) * 0.02 + 0.001
        dt = {"s8": torch.int8, "f16": torch.float16, "f32": torch.float32}[kind]
        o = torch.empty((m, n), dtype=dt, device=dev)
        if kind == "s8":
            extra = dict(bias=torch.randint(-1000, 1001, (n,), dtype=torch.int32, device=dev), relu=True, out_scale=0.05)
        else:
            extra = dict(bias=(torch.rand(n, device=dev) - 0.5).to(dt))
        extra.update(kw)
        us = graph_time_us(torch, lambda: ops.gemm_i8(a, w, out_kind=kind, out=o, scale_a=0.02, scale_w=sw, **extra))
        nbytes = m * k + n * k + m * n * o.element_size()
        out[key] = {"tops": 2.0 * m * n * k / us / 1e6, "us_per_call": us, "gbs": nbytes / us / 1e3,
                    "frac_of_hbm_peak": nbytes / us / 1e3 / peaks["hbm_gbs"], "shape": [m, n, k], "out": kind}
        del a, w, o

    case("i8_linear_k256_s8", 100352, 1024, 256, "s8")
    case("i8_linear_k256_f16", 32768, 4096, 256, "f16")
    case("i8_linear_k256_f16_gelu", 32768, 4096, 256, "f16", activation="gelu")
    case("i8_linear_k256_f32", 32768, 4096, 256, "f32")
    case("i8_linear_8192_f16", 8192, 8192, 8192, "f16")
    return out


def secondary_i8_conv2d(torch, dev):
    """int8 Conv2D (u8 NHWC x s8 HWIO -> s8, bias + Relu, per-channel filter scales) on two layer
    shapes of a ResNet-50 body at batch 32, synthetic values: a 3x3 (gather pass + GEMM) and a 1x1
    (the GEMM reads the activation in place).  TOP/s counts 2 * pixels * OC * KH*KW*IC."""
    from nnops_b200 import ops
    out = {}
    for name, (n, hw, ic, oc, ks, pad) in {"i8_conv2d_3x3_56x56x256": (32, 56, 256, 256, 3, 1),
                                            "i8_conv2d_1x1_56x56x256_to_1024": (32, 56, 256, 1024, 1, 0)}.items():
        x = torch.randint(0, 256, (n, hw, hw, ic), dtype=torch.uint8, device=dev)
        w = torch.randint(-127, 128, (ks, ks, ic, oc), dtype=torch.int8, device=dev)
        sw = torch.rand(oc, device=dev) * 0.01 + 0.005
        bias = torch.randint(-1000, 1001, (oc,), dtype=torch.int32, device=dev)
        o = torch.empty((n, hw, hw, oc), dtype=torch.int8, device=dev)
        ws = torch.empty(1 << 30, dtype=torch.uint8, device=dev)
        packed = ops.prepack_conv2d_i8(w)
        kw = dict(padding=(pad, pad), out_kind="s8", out=o, bias=bias, relu=True, scale_x=0.02, zp_x=128, scale_w=sw,
                  out_scale=0.05, workspace=ws)
        us_raw = graph_time_us(torch, lambda: ops.conv2d_i8(x, w, **kw), calls_per_graph=4, replays=5)
        us_packed = graph_time_us(torch, lambda: ops.conv2d_i8(x, packed, **kw), calls_per_graph=4, replays=5)
        total_ops = 2.0 * n * hw * hw * oc * ks * ks * ic
        out[name] = {"tops": total_ops / us_packed / 1e6, "us_per_call": us_packed, "us_per_call_raw_filter": us_raw,
                     "shape": {"batch": n, "hw": hw, "ic": ic, "oc": oc, "kernel": ks, "padding": pad}}
        del ws
    return out


def run_kernel_only(args):
    """Three launches of one kernel on seeded inputs and nothing else: the command the ncu
    captures under profiles/ are taken from (`--kernel-only i8|gemv|q4gemm|q4gemm2 --shape M N K`)."""
    import torch
    from nnops_b200 import build, capi, ops, synth
    build.build()
    for item in args.knob or []:
        name, _, value = item.partition("=")
        capi.set_knob(name.lower(), int(value))
    m, n, k = args.shape
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(0)
    if args.kernel_only == "quant":
        x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).to(dev)
        scale = torch.full((m,), 0.02, dtype=torch.float32, device=dev)
        zp = torch.zeros(m, dtype=torch.int8, device=dev)
        q = torch.empty((m, k), dtype=torch.int8, device=dev)
        y = torch.empty_like(x)
        for _ in range(3):
            ops.quantize_linear(x, scale, zp, out=q)
            ops.dequantize_linear(q, scale, zp, out=y)
    elif args.kernel_only == "conv":
        # --shape N HW C: batch, plane edge and channel count (in = out) of a 3x3, padding-1 layer.
        n_img, hw, ch = m, n, k
        x = torch.from_numpy(rng.integers(0, 256, (n_img, hw, hw, ch), dtype=np.uint8)).to(dev)
        w = torch.from_numpy(rng.integers(-127, 128, (3, 3, ch, ch), dtype=np.int8)).to(dev)
        sw = torch.from_numpy(rng.uniform(0.005, 0.015, ch).astype(np.float32)).to(dev)
        bias = torch.from_numpy(rng.integers(-1000, 1001, ch).astype(np.int32)).to(dev)
        out = torch.empty((n_img, hw, hw, ch), dtype=torch.int8, device=dev)
        for _ in range(3):
            ops.conv2d_i8(x, w, padding=(1, 1), out_kind="s8", out=out, bias=bias, relu=True, scale_x=0.02, zp_x=128,
                          scale_w=sw, out_scale=0.05)
    elif args.kernel_only == "i8":
        a = torch.from_numpy(synth.s8_uniform(rng, (m, k))).to(dev)
        w = torch.from_numpy(synth.s8_uniform(rng, (n, k))).to(dev)
        sw = torch.from_numpy(rng.uniform(0.001, 0.02, n).astype(np.float32)).to(dev)
        bias = torch.from_numpy(rng.integers(-1000, 1001, n).astype(np.int32)).to(dev)
        out = torch.empty((m, n), dtype=torch.int8, device=dev)
        for _ in range(3):
            ops.gemm_i8(a, w, out_kind="s8", out=out, bias=bias, relu=True, scale_a=0.02, scale_w=sw, out_scale=0.05)
    else:
        wb = torch.from_numpy(synth.q4_1_weights(rng, n, k)).to(dev)
        a = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float16)).to(dev)
        gemv = args.kernel_only == "gemv"
        out = torch.empty((m, n), dtype=torch.float32 if gemv else torch.float16, device=dev)
        for _ in range(3):
            ops.linear_q4_1(a, wb, k, out=out, engine="gemv" if gemv else
                            ("gemm_two_pass" if args.kernel_only == "q4gemm2" else "gemm"))
    torch.cuda.synchronize()
    print(json.dumps({"kernel_only": args.kernel_only, "shape": [m, n, k], "launches": 3}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-secondary", action="store_true", help="skip the Q4_1 and CPU-baseline side measurements")
    ap.add_argument("--reassembly", default="fused", choices=["fused", "multicast", "nccl"],
                    help="N > 1: the GEMM epilogue stores every tile into every rank's output with one peer store per "
                         "rank (fused, the fastest measured), or once through an NVSwitch multicast mapping (multicast; "
                         "falls back to fused where the fabric has none), or NCCL all-gather + interleave kernel (nccl)")
    ap.add_argument("--kernel-only", choices=["i8", "gemv", "q4gemm", "q4gemm2", "quant", "conv"],
                    help="profiling aid: 3 launches of one kernel (q4gemm = fused form, q4gemm2 = two-pass form, "
                         "quant = QuantizeLinear then DequantizeLinear of an [M, K] f32 tensor, per token; N unused; "
                         "conv = int8 3x3 Conv2D, --shape BATCH EDGE CHANNELS)")
    ap.add_argument("--shape", type=int, nargs=3, metavar=("M", "N", "K"), default=[4096, 28672, 8192])
    ap.add_argument("--knob", action="append", metavar="NAME=VALUE",
                    help="set a measurement switch of the library first (e.g. i8_pair=0 for the single-CTA GEMM)")
    args = ap.parse_args()
    if args.kernel_only:
        run_kernel_only(args)
        return
    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch
    import torch.distributed as dist
    from nnops_b200 import build, capi, synth
    from nnops_b200.sharded import ShardedLinearI8, shard_rows

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun for N > 1")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the CUDA library is the only implementation")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    build.build()
    for item in args.knob or []:   # measurement switches, every rank
        name, _, value = item.partition("=")
        capi.set_knob(name.lower(), int(value))
    lib = capi.lib()
    peaks = read_peaks()

    # ---- inputs: identical seeded bytes on every rank; W / scales / bias sharded by rows ----
    c = synth.config5()
    a_host = torch.from_numpy(c.a).pin_memory()
    a = a_host.to(dev)
    w = torch.from_numpy(np.ascontiguousarray(shard_rows(c.w, world, rank))).to(dev)
    layer = ShardedLinearI8(w, n_total=N, world=world, rank=rank, out_kind="s8",
                            bias_shard=torch.from_numpy(np.ascontiguousarray(shard_rows(c.bias, world, rank))).to(dev),
                            scale_w_shard=torch.from_numpy(np.ascontiguousarray(shard_rows(c.scale_w, world, rank))).to(dev),
                            scale_a=c.scale_a, out_scale=c.out_scale, relu=True,
                            mode=args.reassembly if world > 1 else "nccl")
    outs = layer.alloc_outputs(M, count=2)   # fused mode: mapped on every rank through CUDA IPC
    out = outs[0]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident timing: `value` ----
    for _ in range(max(3, args.warmup)):
        layer.forward(a, out)
    barrier()
    uuid = getattr(torch.cuda.get_device_properties(dev), "uuid", None)
    sampler, tight = make_clock_sampler(local_rank, str(uuid) if uuid is not None else None) if rank == 0 else (None, True)
    if rank == 0 and not tight:
        sampler.start()
        time.sleep(0.3)
    k_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = lib.nnb200_launch_count()
    barrier()
    if rank == 0 and tight:
        sampler.start()
    e0.record()
    for i in range(args.steps):
        # Per-launch events around the GEMM itself (the dominant kernel), on the launching stream.
        k_ev[i][0].record()
        layer.local(a, out)
        k_ev[i][1].record()
        layer.reassemble(out)
    e1.record()
    barrier()
    if rank == 0 and tight:
        clocks = sampler.stop()
    launches = lib.nnb200_launch_count() - launches0
    ms_step = max_over_ranks(e0.elapsed_time(e1) / args.steps)
    kernel_ms = max_over_ranks(sum(s.elapsed_time(e) for s, e in k_ev) / args.steps)
    if rank == 0 and not tight:
        time.sleep(0.2)
        clocks = sampler.stop()
    total_ops = 2.0 * M * N * K
    value = total_ops / (ms_step * 1e-3) / 1e12

    # ---- correctness of what was timed: every rank's assembled [M, N] output ----
    # Each rank hashes its own copy; all hashes must agree, and rank 0 compares its copy byte
    # for byte with the reference's CPU route run on the same seeded inputs (all 4096 rows: one
    # call costs the host about a second).
    import hashlib
    out_host_full = out.cpu().numpy()
    my_hash = hashlib.sha256(out_host_full.tobytes()).hexdigest()
    hashes = [my_hash]
    if world > 1:
        hashes = [None] * world
        dist.all_gather_object(hashes, my_hash)
    parity = None
    cpu_full = None
    if rank == 0:
        import oracle
        if oracle.have_ref():
            cpu_full = cpu_reference_run(M, 1, 0, keep_output=True)
            want = cpu_full.pop("output")
            parity = {"rows_checked": M, "equal": bool(np.array_equal(out_host_full, want)),
                      "against": "reference CPU route (oracle/_ref), whole output",
                      "ref_sha256": hashlib.sha256(want.tobytes()).hexdigest()}
        else:
            rows = np.random.default_rng(0).choice(M, 64, replace=False)
            want = oracle.gemm_i8(np.ascontiguousarray(c.a[rows]), c.w, **c.kwargs())
            parity = {"rows_checked": 64, "equal": bool(np.array_equal(out_host_full[rows], want)),
                      "against": "C restatement of the reference arithmetic, sampled rows"}
        parity["ranks_agree"] = len(set(hashes)) == 1
    del out_host_full
    # All ranks learn the verdict and leave together (their buffers are mapped into each other).
    verdict = torch.tensor([1 if (rank != 0 or (parity["equal"] and parity["ranks_agree"])) else 0],
                           dtype=torch.int32, device=dev)
    if world > 1:
        dist.all_reduce(verdict, op=dist.ReduceOp.MIN)
    if int(verdict.item()) == 0:
        if rank == 0:
            print(json.dumps({"error": "parity failure", "parity": parity, "hashes": hashes}), file=sys.stderr, flush=True)
        del out, outs
        layer.close()
        if world > 1:
            dist.destroy_process_group()
        raise SystemExit(1)

    # ---- end to end: host activations in, host result out, every step ----
    # Every step copies its activations from pinned host memory, runs the layer and reads the
    # full result back.  Copies and compute run on three streams over two sets of device/host
    # buffers, so step i's read-back overlaps step i+1's upload and GEMM (PCIe is full duplex).
    # At N > 1 every rank uploads M/g rows of the activations over its own host link and the
    # ranks all-gather the slices over NVLink; every rank reads back only the output columns it
    # produced; together the ranks move the whole input and the whole result once.
    col_lo, col_hi = (0, N) if world == 1 else (layer.col0, layer.col0 + layer.n_per)
    h2d = a_host.numel()
    d2h = M * N
    s_in, s_run, s_back = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    a_dev = [a, torch.empty_like(a)]
    # N > 1: every rank uploads its own M/g rows of the activations over its own host link, then
    # the ranks exchange the slices over NVLink (all-gather in place).
    rows_per = M // world
    row_lo = rank * rows_per
    a_host_slice = a_host[row_lo:row_lo + rows_per] if world > 1 else a_host
    out_dev = outs
    # Each rank's host copy holds only its own columns, densely: a strided pinned destination
    # would make torch fall back to a synchronous host-side copy.
    n_own = col_hi - col_lo
    out_hosts = [torch.empty((M, n_own), dtype=torch.int8).pin_memory() for _ in range(2)]
    own_dense = [torch.empty((M, n_own), dtype=torch.int8, device=dev) for _ in range(2)] if world > 1 else None
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_run = [torch.cuda.Event() for _ in range(2)]
    ev_back = [torch.cuda.Event() for _ in range(2)]

    def e2e_step(i: int):
        b = i & 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_run[b])          # the GEMM that last read this activation buffer
            if world == 1:
                a_dev[b].copy_(a_host, non_blocking=True)
            else:
                a_dev[b][row_lo:row_lo + rows_per].copy_(a_host_slice, non_blocking=True)
            ev_in[b].record()
        with torch.cuda.stream(s_run):
            s_run.wait_event(ev_in[b])
            s_run.wait_event(ev_back[b])        # the read-back that last used this output buffer
            if world > 1:
                # Same stream as the layer's collectives: one communicator.  In place: each rank's
                # input is its own slice of the output.
                dist.all_gather_into_tensor(a_dev[b], a_dev[b][row_lo:row_lo + rows_per])
            # Another rank's previous read-back of this buffer may still be running: order the ranks first.
            layer.forward(a_dev[b], out_dev[b], wait_for_readers=True)
            ev_run[b].record()
        with torch.cuda.stream(s_back):
            s_back.wait_event(ev_run[b])
            if world == 1:
                out_hosts[b].copy_(out_dev[b], non_blocking=True)
            else:
                own_dense[b].copy_(out_dev[b][:, col_lo:col_hi])      # gather this rank's columns on the device
                out_hosts[b].copy_(own_dense[b], non_blocking=True)
            ev_back[b].record()

    for i in range(4):
        e2e_step(i)
    barrier()
    e2e_steps = max(4, min(args.steps, 16))
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(s_in):
        t0.record()
    for i in range(e2e_steps):
        e2e_step(i)
    with torch.cuda.stream(s_back):
        t1.record()
    barrier()
    e2e_ms = max_over_ranks(t0.elapsed_time(t1) / e2e_steps)
    e2e_value = total_ops / (e2e_ms * 1e-3) / 1e12
    e2e_check = bool(torch.equal(out_hosts[0], out_hosts[1]))
    # What the host links give when every rank reads its share back at the same time and nothing
    # else runs: the floor of the end-to-end step (the read-back is its largest transfer).
    src_d2h = own_dense[0] if world > 1 else out_dev[0]
    barrier()
    d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    d0.record()
    for _ in range(4):
        out_hosts[0].copy_(src_d2h, non_blocking=True)
    d1.record()
    barrier()
    d2h_ms = max_over_ranks(d0.elapsed_time(d1) / 4)
    host_link = {"d2h_ms_all_ranks_at_once": d2h_ms, "d2h_gbs_aggregate": d2h / (d2h_ms * 1e-3) / 1e9}

    e2e_matches_resident = None
    if world == 1:
        e2e_matches_resident = hashlib.sha256(out_hosts[0].numpy().tobytes()).hexdigest() == my_hash

    # ---- roofline of the dominant kernel (the tcgen05 GEMM) ----
    derived_peak = 2.0 * peaks["bf16_tflops"]
    per_launch_ops = total_ops / world
    achieved = per_launch_ops / (kernel_ms * 1e-3) / 1e12
    traffic, traffic_source = None, None
    tp = ROOT / "profiles" / "dram_traffic.json"
    if tp.exists() and world == 1:      # captured for the single-GPU launch only
        try:
            traffic = json.loads(tp.read_text()).get("gemm_i8_umma_pair_cfg5_bytes_per_launch")
            traffic_source = ("profiles/dram_traffic.json: dram__bytes_read.sum + dram__bytes_write.sum of one ncu "
                              "capture of this kernel on this workload (profiles/gemm_i8_umma_pair_config5.md); not "
                              "re-measured by this run")
        except (ValueError, OSError):
            traffic = None

    err = capi.take_device_error()
    if world > 1:
        et = torch.tensor([err], dtype=torch.int32, device=dev)
        dist.all_reduce(et, op=dist.ReduceOp.MAX)
        err = int(et.item())
    if err != 0:
        if world > 1:        # every rank leaves, together
            del out, outs, out_dev, a_dev
            layer.close()
            dist.destroy_process_group()
        raise SystemExit(f"device error word = {err}")

    def sampler_factory():
        try:
            return make_clock_sampler(local_rank, str(uuid) if uuid is not None else None)[0]
        except Exception:
            return None

    extra = {}
    cpu_baseline = None
    i8_peak = None
    if rank == 0 and world == 1 and not args.no_secondary:
        # The short side measurements first, the two seconds-long loops under the power cap (the
        # peak probe's and the sustained GEMM's) last: a latency-bound call such as the decode GEMV,
        # timed right after 4.5 s at 990 W, came out at 6.2-6.4 us on some GPUs of this pool and at
        # 4.5 us on the same GPUs when timed first (its time follows the SM clock).
        extra.update(secondary_q4_1(torch, dev, peaks))
        extra.update(secondary_i8_config2(torch, dev, peaks))
        extra.update(secondary_i8_poses(torch, dev))
        extra.update(secondary_i8_conv2d(torch, dev))
        extra.update(secondary_i8_epilogue_bound(torch, dev, peaks))
        extra.update(secondary_quant_linear(torch, dev, peaks))
        extra.update(secondary_i8_decode(torch, dev, peaks, layer.w, layer.kw["scale_w"], layer.kw["bias"]))
        i8_peak = measured_i8_peak(torch, lib, dev, sampler_factory)
        extra["int8_mma_peak"] = i8_peak
        sus = sustained_gemm(torch, layer, a, out, total_ops, sampler_factory)
        sus["frac_of_sustained_int8_peak_random_operands"] = sus["tops"] / i8_peak["sustained_random_operands"]["tops"]
        sus["frac_of_2x_bf16_sustained"] = sus["tops"] / (2.0 * peaks["bf16_tflops_sustained"])
        sus["frac_of_nominal_4500"] = sus["tops"] / 4500.0
        extra["sustained"] = sus
        extra["e2e_op"] = operator_level_bench(10, 3)
        extra["cpu_baseline_q4_1"] = cpu_q4_1_baseline()
        cb = cpu_reference_run(M, 3, 1)
        cpu_baseline = {k: cb[k] for k in ("value", "unit", "cores", "physical_cores", "smt", "kind", "sample")}
        one = None
        try:
            import oracle
            if oracle.have_ref():
                t0 = time.perf_counter()
                oracle.gemm_i8(np.ascontiguousarray(c.a[:256]), c.w, impl="ref", threads=1, **c.kwargs())
                one = 2.0 * 256 * N * K / (time.perf_counter() - t0) / 1e12
        except Exception:
            one = None
        cpu_baseline["one_thread_value"] = one
        cpu_baseline["one_thread_sample"] = "first 256 rows, one call, one thread"
    elif rank == 0 and cpu_full is not None:
        cpu_baseline = {k: cpu_full[k] for k in ("value", "unit", "cores", "physical_cores", "smt", "kind", "sample")}
    if world > 1 and not args.no_secondary:
        # The Q4_1 decode GEMV does not shard in this build: at N > 1 every GPU runs its own
        # replica of the layer (independent requests), and the aggregate is the sum.
        rep = secondary_q4_1(torch, dev, peaks, gemv_only=True)
        mine = [rep["q4_1_gemv_m1"]["gbs"], rep["q4_1_gemv_m8"]["gbs"]]
        allv = [None] * world
        dist.all_gather_object(allv, mine)
        if rank == 0:
            for i, key in enumerate(("q4_1_gemv_m1", "q4_1_gemv_m8")):
                extra[key] = {"gbs": float(sum(v[i] for v in allv)), "per_gpu_gbs": [float(v[i]) for v in allv],
                              "mode": "replicas: one independent GEMV stream per GPU, no exchange",
                              "bytes_per_call": rep[key]["bytes_per_call"]}

    peak = i8_peak["burst_tops"] if i8_peak is not None else derived_peak
    peak_source = ("measured: tcgen05.mma kind::i8 issue-bound probe on this GPU (burst); 2 x measured dense bf16 burst "
                   f"would be {derived_peak:.1f}; nominal dense int8 is 4500") if i8_peak is not None else (
                   f"2 x {peaks['source']} dense bf16 burst ({peaks['bf16_tflops']} TFLOP/s): int8 tensor rate is twice "
                   "the bf16 rate; nominal dense int8 is 4500 (the issue-bound probe runs at N = 1 only)")

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "s8", "data": "synthetic",
            "config": {"workload": WORKLOAD, "m": M, "n": N, "k": K, "shards": world,
                       "reassembly": "none" if world == 1 else (
                           "multicast: GEMM epilogue stores each tile once with multimem.st, the NVSwitch writes it "
                           "into every rank's output; then a device-side flag barrier over peer memory orders the ranks"
                           if layer.multicast_active else (
                               "fused: GEMM epilogue stores each tile into every rank's output over NVLink (P2P), "
                               "then a device-side flag barrier over peer memory orders the ranks"
                               if layer.mode in ("fused", "multicast") else "nccl all-gather + interleave kernel")),
                       "l2": "inputs (268 MB) exceed L2 (126 MB); no flush needed"},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "results_identical_across_buffers": e2e_check,
                    "result_equals_device_resident_run": e2e_matches_resident, "host_link": host_link,
                    "method": "3 streams, double-buffered: H2D of A (at N > 1 each rank uploads M/g rows, then an "
                              "NVLink all-gather), the layer, D2H of each rank's own N/g output columns, every "
                              "step; bytes are totals over the ranks"},
            "gpu_launches": int(launches),
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TOP/s",
                         "frac": achieved / peak, "traffic": traffic, "traffic_source": traffic_source,
                         "peak_source": peak_source, "frac_of_2x_bf16_burst": achieved / derived_peak,
                         "frac_of_nominal_4500": achieved / 4500.0,
                         "kernel": ("gemm_i8_umma_pair_kernel<256,S8> (CTA pairs, tcgen05.mma cta_group::2)" if world == 1
                                    else "gemm_i8_umma_kernel<256,S8,peers> (sharded epilogue)"),
                         "kernel_ms": kernel_ms,
                         "ops_per_launch": per_launch_ops},
            "out_sha256": my_hash, "parity": parity,
            "cpu_baseline": cpu_baseline,
        }
        line.update(extra)
        print(json.dumps(line), flush=True)
    if world > 1:
        # Release the mapped / multicast-bound buffers while every rank is alive.
        del out, outs, out_dev, a_dev
        layer.close()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
