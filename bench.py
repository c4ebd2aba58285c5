#!/usr/bin/env python
"""Benchmark of MIND's deterministic integer BLAS on B200 through the C ABI.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload gemm_i8|gemm_i16|gemm_q16|gemv_q16]
  python bench.py --impl reference ...      # the CPU implementation timed on the host cores

A step is one call of the intrinsic over one set of seeded synthetic operands (the
reference's LCG, generated on the device).  The default workload is the 16384^3 int8 GEMM,
row-sharded over the N ranks (one process per GPU, B replicated, no collective), so the
total work is fixed as N grows.  One JSON line is printed by rank 0.

`value` is timed with operands resident in HBM.  `e2e` is the same product through ONE call
of the intrinsic with HOST operands: at N > 1 rank 0 makes that call with the library
spreading it over the N GPUs itself (mind_b200_set_devices), as the reference's `_mt` entry
points spread one call over the host's cores; the other ranks wait on the host meanwhile.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

KIND_Q16, KIND_I8, KIND_I16 = 0, 1, 2
L2_BYTES = 126 * 1024 * 1024

WORKLOADS = {
    # name: intrinsic, shape, element kind, generator shift, seed (the reference bench's per-shape rule)
    "gemm_i8": dict(fn="matmul_mm_i8_v", m=16384, k=16384, n=16384, kind=KIND_I8, shift=0,
                    seed=0xDEADBEEF00000000 ^ 16384, metric="bit-exact int8 GEMM throughput",
                    unit="TOP/s", dtype="s8 x s8 -> s32", bound="tensor"),
    "gemm_i16": dict(fn="matmul_mm_i16", m=4096, k=4096, n=4096, kind=KIND_I16, shift=0,
                     seed=0xDEADBEEF00000000 ^ 4096, metric="bit-exact int16 GEMM throughput",
                     unit="TOP/s", dtype="s16 x s16 -> s32 (four 8-bit limb products)", bound="tensor"),
    "gemm_q16": dict(fn="matmul_mm_q16_v", m=1024, k=1024, n=1024, kind=KIND_Q16, shift=13,
                     seed=0xDEADBEEF00000000 ^ 1024, metric="bit-exact Q16.16 GEMM throughput",
                     unit="Gop/s", dtype="q16.16 (s32: int8 limb MMAs for a*(b>>16) + (a>>16)*(b&0xffff), fma.rm.f32x2 for the per-product floor of the low halves)",
                     bound="fp32-pipe"),
    "gemv_q16": dict(fn="gemv_q16_mt", m=16384, k=16384, n=1, kind=KIND_Q16, shift=15,
                     seed=0xDEADBEEF00000000 ^ ((16384 << 20) ^ 16384), metric="bit-exact Q16.16 GEMV bandwidth",
                     unit="GB/s", dtype="q16.16 (s32)", bound="hbm"),
    "gemv_i16": dict(fn="matmul_rmajor_i16_v", m=16384, k=16384, n=1, kind=KIND_I16, shift=0,
                     seed=0xDEADBEEF00000000 ^ ((16384 << 20) ^ 16384), metric="bit-exact int16 GEMV bandwidth",
                     unit="GB/s", dtype="s16 x s16 -> s32 (dp2a on byte planes of x)", bound="hbm"),
}
ELEM_BYTES = {KIND_Q16: 4, KIND_I8: 1, KIND_I16: 2}
# dram__bytes_read.sum + dram__bytes_write.sum of the dominant kernel, one launch at the
# workload's full size, from the ncu captures summarised under profiles/ (bytes).
NCU_TRAFFIC = {"gemm_i8": 5699589376 + 1054785280, "gemv_q16": 1073876000 + 3520000,
               "gemm_i16": 96119808 + 46307840, "gemv_i16": 536918272 + 3374848}


def work_units(w, m):
    """Algorithmic work of one call over m rows, in the workload's unit numerator."""
    if w["unit"] == "GB/s":
        es = {KIND_Q16: 4.0, KIND_I8: 1.0, KIND_I16: 2.0}[w["kind"]]
        return es * m * w["k"] + es * w["k"] + 4.0 * m  # matrix once + vector + output, bytes
    return 2.0 * m * w["n"] * w["k"]                       # ops = 2 MKN


def unit_scale(w):
    return {"TOP/s": 1e12, "Gop/s": 1e9, "GB/s": 1e9}[w["unit"]]


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f), "measured"
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []
        self.t_begin, self.t_end = 0.0, float("inf")

    def mark_begin(self):
        self.t_begin = time.perf_counter()

    def mark_end(self):
        self.t_end = time.perf_counter()

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50", "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def wait_ready(self, timeout=6.0):
        """nvidia-smi can take more than a second to print its first sample; the timed region
        is a third of a second, so wait for the sampler before starting the work."""
        t0 = time.perf_counter()
        while self.proc and not self.lines and time.perf_counter() - t0 < timeout:
            time.sleep(0.02)

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def stop(self, spread=False):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        inside = [l for (t, l) in self.lines if self.t_begin <= t <= self.t_end + 0.05]
        window = "timed region"
        if not inside:  # region shorter than one sampling period: fall back to the whole run
            inside, window = [l for (_, l) in self.lines], "whole run (timed region shorter than a sample)"
        for line in inside:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1])); power.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        out = {"sm_mhz": statistics.median(sm) if sm else None,
               "sm_max_mhz": max(mx) if mx else None, "power_w_max": max(power) if power else None,
               "samples": len(sm), "window": window, "reasons": sorted(reasons)}
        if spread and len(sm) >= 5:
            q = sorted(sm)
            out["sm_mhz_p10"], out["sm_mhz_p90"] = q[len(q) // 10], q[(len(q) * 9) // 10]
        return out


# ----------------------------------------------------------------- CPU baseline
def cpu_call(w, a, b, rows, threads=0):
    """One call of the CPU implementation over `rows` rows of the workload's shape."""
    import oracle as O
    k, n = w["k"], w["n"]
    if w["fn"] == "matmul_mm_i8_v":
        return O.baseline_gemm_i8(a, b, rows, k, n, threads)
    if w["fn"] == "matmul_mm_i16":
        return O.baseline_gemm_i16(a, b, rows, k, n, threads)
    if cpu_kind(w) == "reference":
        # the reference's own C dot and thread pool; b is B transposed for the GEMM
        if w["fn"] == "matmul_mm_q16_v":
            return O.reference_gemm_q16_bt(a, b, rows, k, n)
        return O.reference_gemv_q16(a, b, rows, k)
    if w["fn"] == "matmul_mm_q16_v":
        return O.baseline_gemm_q16(a, b, rows, k, n, threads)
    if w["fn"] == "matmul_rmajor_i16_v":
        return O.baseline_gemv_i16(a, b, rows, k, threads)
    return O.baseline_gemv_q16(a, b, rows, k, threads)


def cpu_kind(w):
    """"reference": the Q16.16 workloads are timed on the reference's own compiled C (dot +
    pool, oracle/_ref) when it was built; "port": the threaded restatement (oracle/cpu_baseline.c)."""
    import oracle as O
    return "reference" if w["kind"] == KIND_Q16 and O.ref_lib() is not None else "port"


def cpu_inputs(w, rows):
    import oracle as O
    g = O.Lcg(w["seed"])
    k, n = w["k"], w["n"]
    draw = {KIND_I8: g.i8, KIND_I16: g.i16, KIND_Q16: lambda c: g.q16(c, w["shift"])}[w["kind"]]
    a = draw(rows * k)
    # B follows the WHOLE A in the stream; a fresh generator with its own seed stands in
    # for it here (the CPU timing does not depend on the values).
    g2 = O.Lcg(w["seed"] ^ 0x5555)
    draw2 = {KIND_I8: g2.i8, KIND_I16: g2.i16, KIND_Q16: lambda c: g2.q16(c, w["shift"])}[w["kind"]]
    b = draw2(k * n)
    if cpu_kind(w) == "reference" and n > 1:  # the reference's gate composes the GEMM over B transposed
        b = np.ascontiguousarray(b.reshape(k, n).T).reshape(-1)
    return a, b


def cpu_sample_rows(w, target_s):
    """Rows of the workload whose CPU time is about target_s (time is linear in rows:
    owner-computes row bands), found from one short calibration call."""
    import oracle as O
    cores = O.online_cpus()
    rows0 = min(w["m"], max(4, 64 * min(cores, 256)))  # enough rows per thread to amortise packing B
    a, b = cpu_inputs(w, rows0)
    cpu_call(w, a, b, rows0)  # warm the thread stacks and caches
    t0 = time.perf_counter()
    cpu_call(w, a, b, rows0)
    dt = max(time.perf_counter() - t0, 1e-4)
    rows = int(rows0 * target_s / dt)
    quantum = 4 * min(cores, 256)
    rows = max(quantum, rows // quantum * quantum)
    return min(rows, w["m"]), cores


def cpu_baseline(w, target_s=15.0):
    rows, cores = cpu_sample_rows(w, target_s)
    a, b = cpu_inputs(w, rows)
    t0 = time.perf_counter()
    _, used = cpu_call(w, a, b, rows)
    dt = time.perf_counter() - t0
    return {"value": work_units(w, rows) / dt / unit_scale(w), "unit": w["unit"], "cores": used,
            "kind": cpu_kind(w),
            "sample": f"rows 0..{rows} of {w['m']} (all of K and N), {dt:.2f} s; row bands are independent, so time is linear in rows",
            "host_cpus": cores}


def cpu_baseline_vnni(w, target_s=6.0):
    """The reference's opt-in VNNI rung (MIND_INTDOT=vnni, src/mlir/gemm_tuning.rs:225-236,
    micro-kernel src/mlir/lowering.rs:8186) as a second, labelled CPU figure; None when the host
    has no AVX-512 VNNI."""
    import oracle as O
    if not O.have_vnni():
        return None
    cores = O.online_cpus()
    rows0 = min(w["m"], 64 * min(cores, 256))
    a, b = cpu_inputs(w, rows0)
    O.baseline_gemm_i8_vnni(a, b, rows0, w["k"], w["n"], 0)
    t0 = time.perf_counter()
    O.baseline_gemm_i8_vnni(a, b, rows0, w["k"], w["n"], 0)
    dt = max(time.perf_counter() - t0, 1e-4)
    quantum = 4 * min(cores, 256)
    rows = min(w["m"], max(quantum, int(rows0 * target_s / dt) // quantum * quantum))
    a, b = cpu_inputs(w, rows)
    t0 = time.perf_counter()
    _, used = O.baseline_gemm_i8_vnni(a, b, rows, w["k"], w["n"], 0)
    dt = time.perf_counter() - t0
    return {"value": round(work_units(w, rows) / dt / unit_scale(w), 4), "unit": w["unit"], "cores": used,
            "kind": "port (vpdpbusd rung)"}


def run_reference(args, w):
    """The CPU implementation of the path (threaded port of the reference's kernels,
    oracle/cpu_baseline.c) on the host cores; each step is a bounded row sample."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    per_step = min(10.0, max(0.5, 100.0 / max(1, args.steps + args.warmup)))
    rows, cores = cpu_sample_rows(w, per_step)
    a, b = cpu_inputs(w, rows)
    used = 0
    for _ in range(args.warmup):
        cpu_call(w, a, b, rows)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        _, used = cpu_call(w, a, b, rows)
    dt = time.perf_counter() - t0
    value = work_units(w, rows) * args.steps / dt / unit_scale(w)
    sample = f"rows 0..{rows} of {w['m']} (all of K and N) per step; row bands are independent, so time is linear in rows"
    line = {"impl": "reference", "metric": w["metric"], "value": value, "unit": w["unit"],
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
            "config": {"workload": f"{args.workload} {w['m']}x{w['k']}x{w['n']}", "sample": sample},
            "cpu_baseline": {"value": value, "unit": w["unit"], "cores": used, "kind": cpu_kind(w),
                             "sample": sample, "host_cpus": cores},
            "e2e": {"value": value, "unit": w["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------- GPU arm
def quick_workload(name, blas, torch, stream, dist=None, world=1, rank=0, steps=30, l2="rotate", size=0):
    """Device-resident timing of one of the other benchmark configurations, row-sharded over
    the ranks like the headline workload (each rank its band, max over ranks).  Compact: value,
    unit, kernel_only (the compute kernels without operand re-layout) and its roofline fraction."""
    from mind_b200.shard import row_band
    w = WORKLOADS[name]
    if size:  # the same workload at another (square) size
        w = dict(w, m=size, k=size, n=size)
    m, k, n, kind = w["m"], w["k"], w["n"], w["kind"]
    r0, r1 = row_band(m, world, rank)
    rows = max(r1 - r0, 1)
    tdt = {KIND_Q16: torch.int32, KIND_I8: torch.int8, KIND_I16: torch.int16}[kind]
    a = torch.empty(rows * k, dtype=tdt, device="cuda")
    b = torch.empty(k * n, dtype=tdt, device="cuda")
    c = torch.empty(rows * n, dtype=torch.int32, device="cuda")
    blas.lcg_fill(a, rows * k, kind, w["seed"], r0 * k, w["shift"])
    blas.lcg_fill(b, k * n, kind, w["seed"], m * k, w["shift"])
    fn = getattr(blas, w["fn"])
    sets, flush, _ = operand_sets(torch, a, b, c, l2)
    turn = [0]

    def call():
        pa, pb, pc = sets[turn[0] % len(sets)]
        turn[0] += 1
        if n == 1:
            fn(pa, pb, pc, rows, k)
        else:
            fn(pa, pb, pc, rows, k, n)

    for _ in range(3):
        call()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    blas.profile(True)
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for e0, e1 in evs:
        if flush is not None:
            flush.fill_(1)
        e0.record(stream)
        call()
        e1.record(stream)
    torch.cuda.synchronize()
    n_main, main_ms = blas.profile_read()
    blas.profile(False)
    t = torch.tensor([sum(e0.elapsed_time(e1) for e0, e1 in evs) / steps, main_ms / steps], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, kernel_ms = float(t[0].item()), float(t[1].item())
    scale = unit_scale(w)
    out = {"value": round(work_units(w, m) / (ms * 1e-3) / scale, 2), "unit": w["unit"],
           "kernel_only": round(work_units(w, m) / (kernel_ms * 1e-3) / scale, 2) if n_main and kernel_ms > 0 else None}
    peaks, _ = measured_peaks()
    peak = None
    if w["bound"] == "hbm":
        peak = peaks["hbm_gbs"] * world
    elif w["fn"] == "matmul_mm_i16":
        peak = 2.0 * peaks["bf16_tflops"] / 4.0 * world
    elif w["bound"] == "fp32-pipe":
        peak = fp32_peak(blas) * 2.0 / scale * world   # one FMA per MAC, 2 ops per MAC
    if peak and out["kernel_only"]:
        out["frac"] = round(out["kernel_only"] / peak, 3)
    return out


def operand_sets(torch, a, b, c, mode):
    """How a workload whose operands fit in L2 is kept from finding them there on the next step.
    "rotate": identical copies of (A, B, C), used in turn, larger than L2 together with a margin
    -- the step's inputs are cold, as with inputs larger than L2.  "flush": one set, and a buffer
    twice the size of L2 is written between steps (which also leaves L2 full of dirty lines that
    the step's first kernel then has to write back).  Returns (sets, flush buffer or None, note)."""
    one = a.numel() * a.element_size() + b.numel() * b.element_size() + c.numel() * c.element_size()
    if (a.numel() * a.element_size() + b.numel() * b.element_size()) > 2 * L2_BYTES:
        return [(a, b, c)], None, "operands larger than L2"
    count = max(3, -(-3 * L2_BYTES // one))
    if mode == "flush" or count > 64:  # (a tiny workload would need hundreds of sets: flush instead)
        return [(a, b, c)], torch.empty(2 * L2_BYTES, dtype=torch.uint8, device="cuda"), "L2 flushed between steps"
    sets = [(a, b, c)] + [(a.clone(), b.clone(), torch.empty_like(c)) for _ in range(count - 1)]
    return sets, None, f"{count} operand sets of {one >> 20} MiB used in turn (larger than L2 together)"


_FP64_PEAK = {}


def fp64_peak(blas):
    """Measured FP64 FMA rate of this GPU (FMA / s): a register-only fma.rm.f64 loop inside the
    library, timed with CUDA events (a few ms).  The ceiling of the Q16.16 GEMM in its earlier form
    (one such FMA per product); reported beside the FP32 figure for comparison."""
    if "v" not in _FP64_PEAK:
        _FP64_PEAK["v"] = max(blas.fp64_fma_peak() for _ in range(3))
    return _FP64_PEAK["v"]


def fp32_peak(blas):
    """Measured FP32 FMA rate of this GPU (FMA / s) in the packed round-down form (fma.rm.f32x2,
    register-only loop inside the library, CUDA events).  The Q16.16 GEMM's floor term is one such
    FMA per product, so this is that kernel's ceiling."""
    if "v32" not in _FP64_PEAK:
        _FP64_PEAK["v32"] = max(blas.fp32_fma_peak() for _ in range(3))
    return _FP64_PEAK["v32"]


_CALL_LOOP_C = r"""
#include <stdint.h>
#include <time.h>
typedef int64_t (*fn6_t)(int64_t, int64_t, int64_t, int64_t, int64_t, int64_t);
/* reps back-to-back calls of a six-argument intrinsic, as a compiled caller makes them;
   returns the host seconds spent issuing them (nothing is waited for) */
double call_loop(void *fn, int64_t a, int64_t b, int64_t c, int64_t m, int64_t k, int64_t n, int64_t reps) {
    struct timespec t0, t1;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    for (int64_t i = 0; i < reps; ++i) ((fn6_t)fn)(a, b, c, m, k, n);
    clock_gettime(CLOCK_MONOTONIC, &t1);
    return (double)(t1.tv_sec - t0.tv_sec) + 1e-9 * (double)(t1.tv_nsec - t0.tv_nsec);
}
"""


def compiled_call_loop():
    """A C loop around the entry point (built with gcc into a temporary directory), so that the
    per-call figures of the launch-bound cases are a compiled caller's, without the foreign-call
    overhead of the Python binding.  None when no compiler is at hand."""
    import ctypes as C
    import tempfile
    try:
        d = tempfile.mkdtemp(prefix="mind_b200_bench_")
        src, lib = os.path.join(d, "call_loop.c"), os.path.join(d, "libcall_loop.so")
        with open(src, "w") as f:
            f.write(_CALL_LOOP_C)
        subprocess.run(["gcc", "-O2", "-shared", "-fPIC", "-o", lib, src], check=True, capture_output=True)
        fn = C.CDLL(lib).call_loop
        fn.argtypes, fn.restype = [C.c_void_p] + [C.c_int64] * 7, C.c_double
        return fn
    except Exception:
        return None


def latency_workloads(blas, torch, stream):
    """The launch-latency regime: benchmark configuration 1 (int8 256^3) and the reference's routing
    shape (scores[11922] = catalog[11922 x 384] . query, benches/det_gemv_q16_mt.rs:56-58), device
    resident.  Per call: back-to-back calls on one stream, and the same calls replayed from a CUDA
    graph (32 per graph), which removes the host's launch cost."""
    out = {}

    host_us = {}

    def per_call_us(fn, reps, tag=None):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        t0 = time.perf_counter()
        for _ in range(reps):
            fn()
        t1 = time.perf_counter()  # the host's share: time to enqueue, before anything is waited for
        e1.record(stream)
        torch.cuda.synchronize()
        if tag:
            host_us[tag] = (t1 - t0) * 1e6 / reps
        return e0.elapsed_time(e1) * 1e3 / reps

    def graphed_us(fn, batch=32, reps=20):
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        try:
            with torch.cuda.stream(side):
                blas.set_stream(side.cuda_stream)
                fn()
                torch.cuda.synchronize()
                with torch.cuda.graph(graph, stream=side):
                    for _ in range(batch):
                        fn()
            blas.set_stream(stream.cuda_stream)
            return per_call_us(graph.replay, reps) / batch
        except RuntimeError as ex:  # reported in the line, does not end the bench
            return f"capture failed: {str(ex)[:120]}"
        finally:
            blas.set_stream(stream.cuda_stream)

    n = 256
    seed = 0xDEADBEEF00000000 ^ n
    a = torch.empty(n * n, dtype=torch.int8, device="cuda")
    b = torch.empty(n * n, dtype=torch.int8, device="cuda")
    c = torch.empty(n * n, dtype=torch.int32, device="cuda")
    blas.lcg_fill(a, n * n, KIND_I8, seed, 0, 0)
    blas.lcg_fill(b, n * n, KIND_I8, seed, n * n, 0)
    # the entry point bound once and called with plain integers, as a compiled caller would: the
    # Python wrapper's own argument handling costs about as much as the call
    import ctypes as C
    import mind_b200
    raw = mind_b200.lib().__mind_blas_matmul_mm_i8_v
    pa, pb, pc = C.c_int64(a.data_ptr()), C.c_int64(b.data_ptr()), C.c_int64(c.data_ptr())
    dims = C.c_int64(n)
    call = lambda: raw(pa, pb, pc, dims, dims, dims)
    us, gus = per_call_us(call, 400, "i8"), graphed_us(call)
    r3 = lambda v: round(v, 3) if isinstance(v, float) else v
    out["gemm_i8_256"] = {"us": r3(us), "us_graph": r3(gus), "host_us": r3(host_us["i8"]),
                          "top_s": r3(2.0 * n ** 3 / us / 1e6)}
    loop = compiled_call_loop()
    if loop is not None:  # the same calls from compiled code: one foreign call around the whole loop
        reps = 2000
        fn_addr = C.cast(raw, C.c_void_p)
        loop(fn_addr, a.data_ptr(), b.data_ptr(), c.data_ptr(), n, n, n, 50)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        host_s = loop(fn_addr, a.data_ptr(), b.data_ptr(), c.data_ptr(), n, n, n, reps)
        e1.record(stream)
        torch.cuda.synchronize()
        out["gemm_i8_256"]["us_compiled_caller"] = r3(e0.elapsed_time(e1) * 1e3 / reps)
        out["gemm_i8_256"]["host_us_compiled_caller"] = r3(host_s * 1e6 / reps)

    m, k, q = 11922, 384, 64
    seed = 0xDEADBEEF00000000 ^ ((m << 20) ^ k)
    w = torch.empty(m * k, dtype=torch.int32, device="cuda")
    x = torch.empty(k * q, dtype=torch.int32, device="cuda")
    y = torch.empty(m * q, dtype=torch.int32, device="cuda")
    blas.lcg_fill(w, m * k, KIND_Q16, seed, 0, 15)
    blas.lcg_fill(x, k * q, KIND_Q16, seed, m * k, 15)
    call = lambda: blas.gemv_q16_mt(w, x, y, m, k)
    us, gus = per_call_us(call, 200), graphed_us(call)
    batched = per_call_us(lambda: blas.matmul_mm_q16_v(w, x, y, m, k, q), 50)
    out["gemv_q16_11922x384"] = {"us": r3(us), "us_graph": r3(gus), "us_per_query_64_batched": r3(batched / q)}
    # the int16 row kernel (matmul_rmajor_i16_v) at the GEMV configuration's shape: HBM-bound too
    m = k = 16384
    w16 = torch.empty(m * k, dtype=torch.int16, device="cuda")
    x16 = torch.empty(k, dtype=torch.int16, device="cuda")
    y16 = torch.empty(m, dtype=torch.int32, device="cuda")
    seed = 0xDEADBEEF00000000 ^ ((m << 20) ^ k)
    blas.lcg_fill(w16, m * k, KIND_I16, seed, 0, 0)
    blas.lcg_fill(x16, k, KIND_I16, seed, m * k, 0)
    us = per_call_us(lambda: blas.matmul_rmajor_i16_v(w16, x16, y16, m, k), 30)
    peaks, src = measured_peaks()
    gbs = (2.0 * m * k + 2 * k + 4 * m) / us / 1e3
    out["gemv_i16"] = {"value": round(gbs, 1), "unit": "GB/s", "frac": round(gbs / peaks["hbm_gbs"], 3)}
    return out


def probe_links(max_gpus, up_mib=64, down_mib=128, reps=8):
    """The host-link ceiling that bounds `e2e`: pinned host <-> device copies on 1, 2, 4 ... GPUs at
    once from ONE process (one thread and two streams per GPU, upload and download running
    together, like the library's multi-GPU path), timed with CUDA events per device, slowest
    device counted.  Prints one JSON line per GPU count."""
    import torch
    have = torch.cuda.device_count()
    counts = [g for g in (1, 2, 4, 8, 16) if g <= min(max_gpus, have)]
    for g in counts:
        results = [None] * g
        ready = threading.Barrier(g)

        def work(d):
            torch.cuda.set_device(d)
            hin = torch.empty(up_mib << 20, dtype=torch.uint8).pin_memory()
            hout = torch.empty(down_mib << 20, dtype=torch.uint8).pin_memory()
            din = torch.empty(up_mib << 20, dtype=torch.uint8, device=f"cuda:{d}")
            dout = torch.empty(down_mib << 20, dtype=torch.uint8, device=f"cuda:{d}")
            s_up, s_down = torch.cuda.Stream(d), torch.cuda.Stream(d)
            out = {}
            for mode in ("up", "down", "both"):
                for timed in (False, True):
                    torch.cuda.synchronize(d)
                    ready.wait()
                    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
                    ev[0].record(s_up); ev[2].record(s_down)
                    for _ in range(reps if timed else 1):
                        if mode != "down":
                            with torch.cuda.stream(s_up):
                                din.copy_(hin, non_blocking=True)
                        if mode != "up":
                            with torch.cuda.stream(s_down):
                                hout.copy_(dout, non_blocking=True)
                    ev[1].record(s_up); ev[3].record(s_down)
                    torch.cuda.synchronize(d)
                    if timed:
                        out[mode] = max(ev[0].elapsed_time(ev[1]), ev[2].elapsed_time(ev[3])) / reps
            results[d] = out

        threads = [threading.Thread(target=work, args=(d,)) for d in range(g)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        line = {"probe": "pinned host link", "gpus": g, "up_mib_per_gpu": up_mib, "down_mib_per_gpu": down_mib}
        for mode, nbytes in (("up", up_mib), ("down", down_mib), ("both", up_mib + down_mib)):
            worst = max(r[mode] for r in results)
            line[f"{mode}_ms"] = round(worst, 3)
            line[f"{mode}_gb_s_aggregate"] = round(g * (nbytes << 20) / (worst * 1e-3) / 1e9, 1)
        print(json.dumps(line), flush=True)


def whole_output_gate(w, blas, torch, a, b, c, rows, k, n, rank, path=0):
    """Byte-identity gate on the WHOLE output of this rank before any timing (the reference's
    benches compare the whole output with their scalar oracle, benches/det_matmul_i8.rs:310-352;
    an O(N^3) CPU oracle is too slow at these sizes):
      int8 / int16 GEMM  exact Freivalds check in Z/2^32, C.v == A.(B.v) for two random vectors
                         (both sides are exact sums mod 2^32, so equality is not probabilistic in
                         the arithmetic, only in the choice of v), plus end rows against the oracle;
      Q16.16 GEMM        the whole matrix against the independent all-integer kernel (path 1),
                         plus end rows against the oracle (the rule is not bilinear);
      GEMV               every output against the CPU oracle."""
    import oracle as O
    es = ELEM_BYTES[w["kind"]]
    if n == 1:
        want = (O.gemv_i16 if w["kind"] == KIND_I16 else O.gemv_q16)(a.cpu().numpy(), b.cpu().numpy(), rows, k)
        if not np.array_equal(c[:rows].cpu().numpy(), want):
            raise SystemExit(f"rank {rank}: GEMV output differs from the oracle; not timing a wrong kernel")
        return "every output vs the CPU oracle"
    bh = b.cpu().numpy()
    oracle_fn = {"matmul_mm_i8_v": O.gemm_i8, "matmul_mm_i16": O.gemm_i16, "matmul_mm_q16_v": O.gemm_q16}[w["fn"]]
    for s0 in (0, rows - 2):
        ah = a[s0 * k:(s0 + 2) * k].cpu().numpy()
        if not np.array_equal(c[s0 * n:(s0 + 2) * n].cpu().numpy(), oracle_fn(ah, bh, 2, k, n)):
            raise SystemExit(f"rank {rank}: rows {s0}..{s0 + 2} of this band differ from the oracle; not timing a wrong kernel")
    if w["kind"] == KIND_Q16:
        c2 = torch.empty_like(c)
        blas.set_gemm_path(1)
        blas.matmul_mm_q16_v(a, b, c2, rows, k, n)
        blas.synchronize()
        blas.set_gemm_path(path)
        if not torch.equal(c[: rows * n], c2[: rows * n]):
            raise SystemExit(f"rank {rank}: Q16.16 GEMM differs from the all-integer kernel")
        return "whole C vs the all-integer kernel + end rows vs the CPU oracle"
    gen = torch.Generator(device="cuda").manual_seed(1234 + rank)
    for _ in range(2):
        v = torch.randint(-2**31, 2**31 - 1, (n,), dtype=torch.int64, device="cuda", generator=gen).to(torch.int32)
        bv = torch.empty(k, dtype=torch.int32, device="cuda")
        abv = torch.empty(rows, dtype=torch.int32, device="cuda")
        cv = torch.empty(rows, dtype=torch.int32, device="cuda")
        blas.matvec_wrap(b, es, k, n, v, bv)
        blas.matvec_wrap(a, es, rows, k, bv, abv)
        blas.matvec_wrap(c, 4, rows, n, v, cv)
        blas.synchronize()
        if not torch.equal(abv, cv):
            raise SystemExit(f"rank {rank}: C.v != A.(B.v) mod 2^32; not timing a wrong kernel")
    return "exact Freivalds in Z/2^32 over the whole C (2 vectors) + end rows vs the CPU oracle"


def output_hash(torch, dist, c, m, n, world, rank, r0, rows):
    """sha256 of C that does not depend on the rank count: every rank hashes its band in blocks of
    ceil(M / 8) rows (a band of 1, 2, 4 or 8 ranks is a whole number of them), rank 0 hashes the
    block digests in row order.  Outside every timed region."""
    block = -(-m // 8)
    if rows % block and r0 + rows != m:
        return None
    host = c[: rows * n].cpu().numpy()
    digests = b"".join(hashlib.sha256(host[i * n:min(i + block, rows) * n].tobytes()).digest()
                       for i in range(0, rows, block))
    if world > 1:
        parts = [None] * world
        dist.all_gather_object(parts, digests)
        digests = b"".join(parts)
    return hashlib.sha256(digests).hexdigest()


def run_mine(args, w):
    import torch
    import torch.distributed as dist

    from mind_b200 import blas
    from mind_b200.shard import row_band

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    host_group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        host_group = dist.new_group(backend="gloo")  # waits on the host: no kernel spins on a GPU meanwhile
    if blas.device_count() == 0:
        raise SystemExit("libmind_b200 found no sm_100 device; there is no fallback to time")
    stream = torch.cuda.current_stream()
    blas.set_stream(stream.cuda_stream)
    blas.set_gemm_path(args.path)
    if args.group_m or args.raster:
        blas.set_tile_order(args.group_m, args.raster)

    m, k, n, kind = w["m"], w["k"], w["n"], w["kind"]
    es = ELEM_BYTES[kind]
    r0, r1 = row_band(m, world, rank)
    rows = r1 - r0
    tdt = {KIND_Q16: torch.int32, KIND_I8: torch.int8, KIND_I16: torch.int16}[kind]
    # This rank's band of A, all of B (replicated), this rank's band of C.
    a = torch.empty(max(rows * k, 1), dtype=tdt, device="cuda")
    b = torch.empty(k * n, dtype=tdt, device="cuda")
    c = torch.empty(max(rows * n, 1), dtype=torch.int32, device="cuda")
    blas.lcg_fill(a, rows * k, kind, w["seed"], r0 * k, w["shift"])
    blas.lcg_fill(b, k * n, kind, w["seed"], m * k, w["shift"])
    fn = getattr(blas, w["fn"])

    def step(pa, pb, pc, nrows=rows):
        if n == 1:
            fn(pa, pb, pc, nrows, k)
        else:
            fn(pa, pb, pc, nrows, k, n)

    # Byte-identity gate before any timing, and the hash of the whole C.
    step(a, b, c)
    blas.synchronize()
    gate = "skipped (--no-check)"
    c_sha = None
    if rows >= 2 and not args.no_check:
        gate = whole_output_gate(w, blas, torch, a, b, c, rows, k, n, rank, args.path)
        c_sha = output_hash(torch, dist, c, m, n, world, rank, r0, rows)

    in_bytes = (rows * k + k * n) * es
    # operands that could sit in L2 between steps: several sets used in turn (or a flush)
    sets, flush, l2_note = operand_sets(torch, a, b, c, args.l2)
    turn = [0]

    def next_set():
        turn[0] += 1
        return sets[turn[0] % len(sets)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()  # nvidia-smi takes a moment to come up: start it before the warm-up
        sampler.wait_ready()
    for _ in range(args.warmup):
        if flush is not None:
            flush.fill_(1)
        step(*next_set())
    barrier()
    sampler.mark_begin()
    launches0 = blas.kernel_launches()
    blas.profile(True)
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    for e0, e1 in evs:
        if flush is not None:
            flush.fill_(1)
        e0.record(stream)
        step(*next_set())
        e1.record(stream)
    barrier()
    sampler.mark_end()
    launches = blas.kernel_launches() - launches0
    n_main, main_ms = blas.profile_read()
    blas.profile(False)
    clocks = sampler.stop() if rank == 0 else None
    ms = sum(e0.elapsed_time(e1) for e0, e1 in evs)
    t = torch.tensor([ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())

    # Sustained leg: the same call back to back for some seconds (the timed region above is a
    # burst of tens of milliseconds, over before the power cap bites), with the SM clock sampled
    # throughout.  time x clock (cycles per step) compares runs on boxes with different caps.
    sustained = None
    if args.sustain > 0:
        est = max(ms_total / args.steps, 1e-3)
        reps = max(10, int(args.sustain * 1e3 / est))
        s2 = ClockSampler(local)
        if rank == 0:
            s2.start()
            s2.wait_ready()
        barrier()
        s2.mark_begin()
        y0, y1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        y0.record(stream)
        for _ in range(reps):
            step(*next_set())
        y1.record(stream)
        barrier()
        s2.mark_end()
        t = torch.tensor([y0.elapsed_time(y1)], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        sus_ms = float(t.item())
        if rank == 0:
            ck = s2.stop(spread=True)
            per = sus_ms / reps
            sustained = {"seconds": round(sus_ms * 1e-3, 2), "steps": reps,
                         "value": round(work_units(w, m) * reps / (sus_ms * 1e-3) / unit_scale(w), 1), "unit": w["unit"],
                         "ms_per_step": round(per, 4), "sm_mhz_median": ck.get("sm_mhz"), "sm_mhz_p10": ck.get("sm_mhz_p10"),
                         "sm_mhz_p90": ck.get("sm_mhz_p90"), "clock_samples": ck.get("samples"),
                         "power_w_max": ck.get("power_w_max"), "reasons": ck.get("reasons"),
                         "mcycles_per_step": round(per * 1e-3 * ck["sm_mhz"], 3) if ck.get("sm_mhz") else None,
                         "l2": l2_note}

    # End to end: the same product through ONE call with HOST (pinned) operands, so every step
    # copies A and B to the device(s) and C back inside the timed region.  At N > 1 rank 0 makes
    # the call and the library spreads it over the N GPUs (row bands, as the ranks above); the
    # other ranks wait on the host.
    e2e = e2e_pageable = None
    e2e_steps = max(1, min(args.steps, 3))
    del flush
    del sets[1:]
    if world > 1:
        dist.barrier(group=host_group)
    if rank == 0:
        if world == 1:
            ha = torch.empty(a.numel(), dtype=tdt).pin_memory(); ha.copy_(a)
            full_a = a
        else:
            # the whole A on the host: generated band by band on this rank's GPU
            ha = torch.empty(m * k, dtype=tdt).pin_memory()
            band = -(-m // world)
            tmp = torch.empty(band * k, dtype=tdt, device="cuda")
            for s0 in range(0, m, band):
                nr = min(band, m - s0)
                blas.lcg_fill(tmp, nr * k, kind, w["seed"], s0 * k, w["shift"])
                blas.synchronize()
                ha[s0 * k:(s0 + nr) * k].copy_(tmp[: nr * k])
            del tmp
        hb = torch.empty(b.numel(), dtype=tdt).pin_memory(); hb.copy_(b)
        hc = torch.empty(m * n, dtype=torch.int32).pin_memory()
        blas.set_devices(world)

        def timed_calls(pa, pb, pc, reps):
            step(pa, pb, pc, m)  # warm-up (sizes the staging buffers, starts the device threads)
            torch.cuda.synchronize()
            x0, x1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            x0.record(stream)
            for _ in range(reps):
                step(pa, pb, pc, m)  # synchronous: returns when C is back in host memory
            x1.record(stream)
            torch.cuda.synchronize()
            return x0.elapsed_time(x1) * 1e-3 / reps

        per_call = timed_calls(ha, hb, hc, e2e_steps)
        total_work = work_units(w, m)
        e2e = {"value": total_work / per_call / unit_scale(w), "unit": w["unit"],
               "h2d_bytes_per_step": (m * k + k * n) * es, "d2h_bytes_per_step": m * n * 4,
               "steps": e2e_steps, "ms_per_step": round(per_call * 1e3, 3),
               "how": "one call, pinned host operands" + (f", spread over {world} GPUs by the library" if world > 1 else "")}
        if world == 1:
            if not torch.equal(hc[: rows * n], c[: rows * n].cpu()):
                raise SystemExit("host-pointer call and device-pointer call disagree")
        else:
            hc_band = hc[r0 * n:(r0 + rows) * n]
            if not torch.equal(hc_band, c[: rows * n].cpu()):
                raise SystemExit("the multi-GPU host call disagrees with rank 0's device band")
            if c_sha is not None:
                block = -(-m // 8)
                dig = b"".join(hashlib.sha256(hc[i * n:min(i + block, m) * n].numpy().tobytes()).digest()
                               for i in range(0, m, block))
                if hashlib.sha256(dig).hexdigest() != c_sha:
                    raise SystemExit("the multi-GPU host call's C does not hash like the ranks' C")
        if not args.no_pageable:
            # the same call with ordinary (pageable) heap buffers, what a Vec / malloc caller passes
            pa, pb = ha.numpy().copy(), hb.numpy().copy()
            pc = np.empty(m * n, dtype=np.int32)
            per_call = timed_calls(pa, pb, pc, 1 if per_call > 0.05 else 2)
            if not np.array_equal(pc, hc.numpy()):
                raise SystemExit("pageable-host call and pinned-host call disagree")
            e2e_pageable = {"value": round(total_work / per_call / unit_scale(w), 2), "unit": w["unit"],
                            "ms_per_step": round(per_call * 1e3, 2)}
            del pa, pb, pc
        blas.set_devices(1)
        del ha, hb, hc
    if world > 1:
        dist.barrier(group=host_group)

    # Optional: the rank-ordered all-gather of the C bands over NCCL (not part of `value`: the
    # path needs no collective; reported so that "with the gather" can be read off too).
    gather_ms = None
    if world > 1 and args.gather and n > 1:
        from mind_b200.shard import all_gather_rows
        full = None
        for _ in range(2):
            full = all_gather_rows(c[: rows * n], m, n)
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record(stream)
        for _ in range(5):
            full = all_gather_rows(c[: rows * n], m, n)
        g1.record(stream)
        torch.cuda.synchronize()
        t = torch.tensor([g0.elapsed_time(g1) / 5], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        gather_ms = float(t.item())
        if not torch.equal(full[r0:r1].reshape(-1), c[: rows * n]):
            raise SystemExit(f"rank {rank}: gathered C does not hold this rank's band")
        del full

    # The metric also names the Q16.16 GEMM, the GEMV and (by config) the int16 GEMM: their
    # device-resident numbers ride along, row-sharded over the ranks like the headline workload.
    others = None
    if args.workload == "gemm_i8" and not args.size and not args.no_others:
        del a, b, c
        torch.cuda.empty_cache()
        others = {name: quick_workload(name, blas, torch, stream, dist, world, rank, l2=args.l2)
                  for name in ("gemm_q16", "gemv_q16", "gemm_i16")}
        # (cfg 2 is 1024^3, where set-up and two tile epilogues are a third of the kernel: the same at 4096^3)
        others["gemm_q16_4096"] = quick_workload("gemm_q16", blas, torch, stream, dist, world, rank, steps=10,
                                                 l2=args.l2, size=4096)
        if world == 1:
            others.update(latency_workloads(blas, torch, stream))

    if rank == 0:
        peaks, peak_src = measured_peaks()
        scale = unit_scale(w)
        total_work = work_units(w, m)  # whole job: every rank's rows
        value = total_work * args.steps / (ms_total * 1e-3) / scale
        per_launch = work_units(w, rows)
        # main_ms sums the call's compute kernels (one per call, two for the Q16.16 hybrid)
        achieved = per_launch * args.steps / (main_ms * 1e-3) / scale if n_main and main_ms > 0 else None
        if w["bound"] == "hbm":
            peak, peak_note = peaks["hbm_gbs"], f"{peak_src} STREAM-style copy"
        elif w["bound"] == "tensor":
            # no int8 figure is measured on this pool: the int8 tensor rate is twice bf16
            peak, peak_note = 2.0 * peaks["bf16_tflops"], f"2 x {peak_src} cuBLAS bf16 burst"
            if w["fn"] == "matmul_mm_i16":
                peak, peak_note = peak / 4.0, peak_note + " / 4 limb products"
        else:
            peak = 2.0 * fp32_peak(blas) / scale
            peak_note = "measured here: register-only fma.rm.f32x2 loop (one FP32 FMA per product, 2 ops)"
        roofline = {"bound": w["bound"], "achieved": achieved, "peak": peak, "unit": w["unit"],
                    "frac": (achieved / peak) if achieved and peak else None,
                    "traffic": NCU_TRAFFIC.get(args.workload) if not args.size and world == 1 else None,
                    "kernel": "gemm_tc_kernel" if w["bound"] == "tensor" else ("rows_group_kernel" if w["bound"] == "hbm" else "gemm_q16_fused_kernel"),
                    "kernel_ms": main_ms / args.steps if n_main else None, "peak_source": peak_note}
        if w["bound"] == "fp32-pipe" and achieved:
            # the ceiling of the earlier form of this kernel (one fma.rm.f64 per product), for comparison
            roofline["frac_of_fp64_fma_peak"] = achieved / (2.0 * fp64_peak(blas) / scale)
        if w["bound"] == "tensor":
            roofline["frac_of_nominal_4500"] = achieved / (4500.0 / (4.0 if w["fn"] == "matmul_mm_i16" else 1.0)) if achieved else None
            if sustained:
                # the sustained leg against the sustained cuBLAS figure (same regime on both sides)
                div = 4.0 if w["fn"] == "matmul_mm_i16" else 1.0
                sustained["frac_of_sustained_peak"] = round(sustained["value"] / world / (2.0 * peaks["bf16_tflops_sustained"] / div), 3)
                sustained["frac_of_nominal_4500"] = round(sustained["value"] / world / (4500.0 / div), 3)
        # Key order: the contract's keys first; the compact extras go LAST, so that a reader who
        # keeps only the end of the line still sees them whole.
        line = {"metric": w["metric"], "value": value, "unit": w["unit"], "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_total / args.steps,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": w["dtype"], "data": "synthetic"}
        line["config"] = {"workload": f"{args.workload} {m}x{k}x{n}" if n > 1 else f"{args.workload} {m}x{k}",
                          "sharding": f"{world} row band(s) of {-(-m // world)} rows, B replicated, no collective",
                          "l2": l2_note,
                          "gemm_path": args.path, "seed": hex(w["seed"]), "gate": gate}
        line["roofline"] = roofline
        line["cpu_baseline"] = cpu_baseline(w) if world == 1 and not args.no_cpu else None
        line["clocks"] = clocks
        line["e2e"] = e2e
        line["gpu_launches"] = launches
        if gather_ms is not None:
            line["all_gather_c"] = {"ms": gather_ms, "bytes_received_per_rank": m * n * 4,
                                    "note": "NCCL all-gather of the C row bands, rank order; outside `value`"}
        if line["cpu_baseline"] and w["fn"] == "matmul_mm_i8_v":
            line["cpu_baseline_vnni"] = cpu_baseline_vnni(w)
        if e2e_pageable is not None:
            line["e2e_pageable"] = e2e_pageable
        line["c_sha256"] = c_sha
        if sustained is not None:
            for drop in ("steps", "clock_samples", "l2", "unit"):
                sustained.pop(drop, None)
            line["sustained"] = sustained
        if others is not None:
            line["other_workloads"] = others
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier(group=host_group)
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="mine", choices=["mine", "reference"])
    ap.add_argument("--workload", default="gemm_i8", choices=sorted(WORKLOADS))
    ap.add_argument("--path", type=int, default=0, help="0: auto, 2: CTA pairs, 3: one CTA per tile, 1: CUDA cores")
    ap.add_argument("--size", type=int, default=0, help="override M = K (= N) for quick runs")
    ap.add_argument("--sustain", type=float, default=3.0, help="seconds of back-to-back calls after the timed region (0: skip)")
    ap.add_argument("--group-m", type=int, default=0, help="int8 tile order: m-tiles per group (0: default)")
    ap.add_argument("--raster", type=int, default=0, help="int8 tile order variant (0: default)")
    ap.add_argument("--l2", default="rotate", choices=["rotate", "flush"],
                    help="operands that fit in L2: use several operand sets in turn (default) or flush L2 between steps")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-check", action="store_true", help="skip the whole-output gate before timing")
    ap.add_argument("--no-others", action="store_true", help="skip the other configurations' ride-along numbers")
    ap.add_argument("--no-pageable", action="store_true", help="skip the pageable-host end-to-end call")
    ap.add_argument("--gather", action="store_true", help="N > 1: also time the optional all-gather of C")
    ap.add_argument("--probe-links", type=int, default=0, metavar="G",
                    help="instead of the bench: pinned host<->device copy ceiling on 1, 2, 4 ... G GPUs at once")
    args = ap.parse_args()
    if args.probe_links:
        probe_links(args.probe_links)
        return
    if args.warmup < 3:
        args.warmup = 3
    w = dict(WORKLOADS[args.workload])
    if args.size:
        w["m"] = w["k"] = args.size
        if w["n"] > 1:
            w["n"] = args.size
    if args.impl == "reference":
        run_reference(args, w)
    else:
        run_mine(args, w)


if __name__ == "__main__":
    main()
