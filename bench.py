#!/usr/bin/env python
"""Benchmark of the GEMM hot path on B200: one JSON line per run.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl b200|reference]

Headline workload (default): HGEMM, row-major, A not transposed, B transposed, M = N = K = 8192, alpha 1, beta 0,
A and B ~ 0.1*N(0,1) in fp16, C poisoned with NaN. A step is one clblast::Gemm call through the C ABI.
With N > 1 GPUs (one process per GPU under torchrun) the problem grows with N (weak scaling): C is M = 8192*N rows,
each rank owns the 8192 rows of A and C of its block and needs all of B, which rank 0 re-sends inside every timed step:
a binomial tree of copy-engine copies over NVLink (clblast_b200.multi_gpu.CopyEngineFanout) that overlaps the previous
step's GEMM and takes no SM from it (`--bcast nccl` selects an NCCL broadcast instead). `value` is TFLOPS =
2*M*N*K / t over all ranks, t the max over ranks of the device time measured with CUDA events. `e2e` repeats the
measurement through the API with pinned host buffers: host->device copies of the inputs and the device->host copy
of C are inside the timed region.

Further keys of the line: `roofline` (dominant kernel alone, against the measured peak), `sustained`, `sweep` (every
other single-GPU configuration with its own roofline entry), `sync_api` (wall clock around the host-synchronous
public call), `peaks` (library GEMMs measured in this run as denominators for the precisions MEASURED_PEAKS.json
lacks), `sharded` (the two column-sharded problems at this N, strong scaling), `reference_b200` (the reference's
own CUDA build on the same GPU where it has been built), `cpu_baseline`.

`--impl reference` times the CPU restatement of the reference's kernels (the oracle port; the reference itself has
no CPU path without an OpenCL runtime) on a bounded sample of the same workload, on all host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

ROW, COL, NO, YES = 101, 102, 111, 112
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}

# name -> description of one step. kind: gemm | strided | conv | sharded
WORKLOADS = {
    "hgemm_8192": dict(kind="gemm", precision=16, layout=ROW, ta=NO, tb=YES, m=8192, n=8192, k=8192, alpha=1.0,
                       beta=0.0, dist="normal0.1", bound="tensor"),
    "hgemm_16384x4096x8192": dict(kind="gemm", precision=16, layout=ROW, ta=NO, tb=YES, m=16384, n=4096, k=8192,
                                  alpha=1.0, beta=0.0, dist="normal0.1", bound="tensor"),
    "sgemm_8192": dict(kind="gemm", precision=32, layout=COL, ta=NO, tb=NO, m=8192, n=8192, k=8192, alpha=1.5,
                       beta=0.5, ld_pad=16, dist="uniform1", bound="fp32"),
    "sgemm_4096": dict(kind="gemm", precision=32, layout=COL, ta=NO, tb=NO, m=4096, n=4096, k=4096, alpha=1.5,
                       beta=0.5, ld_pad=16, dist="uniform1", bound="fp32"),
    "sgemm_2048": dict(kind="gemm", precision=32, layout=COL, ta=NO, tb=NO, m=2048, n=2048, k=2048, alpha=1.5,
                       beta=0.5, ld_pad=16, dist="uniform1", bound="fp32"),
    "sgemm_1000": dict(kind="gemm", precision=32, layout=COL, ta=NO, tb=NO, m=1000, n=1000, k=1000, alpha=1.5,
                       beta=0.5, ld_pad=16, dist="uniform1", bound="fp32"),
    "sgemm_1024": dict(kind="gemm", precision=32, layout=ROW, ta=NO, tb=NO, m=1024, n=1024, k=1024, alpha=0.7,
                       beta=0.3, dist="uniform1", bound="fp32"),
    "sgemm_ragged": dict(kind="gemm", precision=32, layout=COL, ta=NO, tb=NO, m=4097, n=3071, k=1025, alpha=1.5,
                         beta=0.5, ld_pad=16, dist="uniform1", bound="fp32"),
    "dgemm_8192": dict(kind="gemm", precision=64, layout=COL, ta=NO, tb=NO, m=8192, n=8192, k=8192, alpha=1.0,
                       beta=0.0, dist="uniform1", bound="fp64"),
    # One large column-major GEMM sharded by column blocks of C over the ranks (strong scaling); A is re-sent from
    # rank 0 in every step, B and C blocks are resident on their ranks.
    "dgemm_32768_sharded": dict(kind="sharded", precision=64, layout=COL, ta=NO, tb=NO, m=32768, n=32768, k=32768,
                                alpha=1.0, beta=0.0, dist="uniform1", bound="fp64"),
    "sgemm_65536_sharded": dict(kind="sharded", precision=32, layout=COL, ta=NO, tb=NO, m=65536, n=65536, k=65536,
                                alpha=1.0, beta=0.0, dist="uniform1", bound="fp32"),
    "sgemm_16384_sharded": dict(kind="sharded", precision=32, layout=COL, ta=NO, tb=NO, m=16384, n=16384, k=16384,
                                alpha=1.0, beta=0.0, dist="uniform1", bound="fp32"),
    "batched_32": dict(kind="strided", precision=32, layout=COL, ta=NO, tb=NO, m=32, n=32, k=32, batch=8192,
                       alpha=1.0, beta=1.0, dist="uniform1", bound="hbm"),
    "batched_64x128x96": dict(kind="strided", precision=32, layout=COL, ta=NO, tb=NO, m=64, n=128, k=96, batch=2048,
                              alpha=1.0, beta=1.0, dist="uniform1", bound="hbm"),
    # larger problems per batch entry run on the tensor cores (batch as third tensor-map dimension)
    "hgemm_batched_1024x64": dict(kind="strided", precision=16, layout=ROW, ta=NO, tb=YES, m=1024, n=1024, k=1024,
                                  batch=64, alpha=1.0, beta=0.0, dist="normal0.1", bound="tensor"),
    "sgemm_batched_512x128": dict(kind="strided", precision=32, layout=COL, ta=NO, tb=NO, m=512, n=512, k=512,
                                  batch=128, alpha=1.0, beta=0.0, dist="uniform1", bound="fp32"),
    # the next rows of the path: complex GEMM on the real tensor-core kernels, rank-k update, triangular solve
    "cgemm_4096": dict(kind="gemm", precision=3232, layout=COL, ta=NO, tb=NO, m=4096, n=4096, k=4096, alpha=1.5,
                       beta=0.5, dist="uniform1", bound="fp32"),
    "syrk_8192": dict(kind="syrk", precision=32, layout=COL, n=8192, k=8192, alpha=1.0, beta=0.0, dist="uniform1",
                      bound="fp32"),
    "trsm_8192": dict(kind="trsm", precision=32, layout=COL, m=8192, n=8192, alpha=1.0, dist="uniform1", bound="fp32"),
    "conv_56": dict(kind="conv", precision=32, channels=64, height=56, width=56, kh=3, kw=3, pad=1, stride=1, dil=1,
                    num_kernels=128, batch=32, bound="fp32"),
    # the same convolution in half (implicit GEMM, im2col matrix in tensor memory) and double precision (im2col into
    # scratch, then the FP64 tensor-core GEMM)
    "hconv_56": dict(kind="conv", precision=16, channels=64, height=56, width=56, kh=3, kw=3, pad=1, stride=1, dil=1,
                     num_kernels=128, batch=32, bound="tensor"),
    "dconv_56": dict(kind="conv", precision=64, channels=64, height=56, width=56, kh=3, kw=3, pad=1, stride=1, dil=1,
                     num_kernels=128, batch=32, bound="fp64"),
}
SHARDED_IN_EVERY_RUN = ("dgemm_32768_sharded", "sgemm_65536_sharded")
TORCH_DT = {16: "float16", 32: "float32", 64: "float64", 3232: "complex64"}
ELEM = {16: 2, 32: 4, 64: 8, 3232: 8}
DTYPE_NAME = {16: "f16", 32: "f32", 64: "f64", 3232: "c32"}
# ncu summaries whose "`roofline.traffic` for bench.py: <bytes> bytes per launch." line feeds roofline.traffic
PROFILE_OF = {"hgemm_8192": "hgemm_tc_pair_kernel__hgemm_8192.md"}


def flops_of(w, scale_m=1):
    if w["kind"] in ("gemm", "sharded"):
        return (8.0 if w["precision"] > 100 else 2.0) * w["m"] * scale_m * w["n"] * w["k"]
    if w["kind"] == "syrk":
        return 1.0 * w["n"] * (w["n"] + 1) * w["k"]       # one triangle of n x n outputs, 2k flops each
    if w["kind"] == "trsm":
        return 1.0 * w["m"] * w["m"] * w["n"]             # left side: m^2 n
    if w["kind"] == "strided":
        return 2.0 * w["m"] * w["n"] * w["k"] * w["batch"] * scale_m
    oh = (w["height"] + 2 * w["pad"] - w["dil"] * (w["kh"] - 1) - 1) // w["stride"] + 1
    ow = (w["width"] + 2 * w["pad"] - w["dil"] * (w["kw"] - 1) - 1) // w["stride"] + 1
    return 2.0 * w["batch"] * scale_m * oh * ow * w["num_kernels"] * w["channels"] * w["kh"] * w["kw"]


def min_bytes_of(w):
    """Algorithmic bytes of one launch: every operand read once, C written once (and read once when beta != 0)."""
    e = ELEM[w["precision"]]
    if w["kind"] in ("gemm", "sharded"):
        m, n, k = w["m"], w["n"], w["k"]
        return e * (m * k + k * n + m * n * (2 if w["beta"] != 0 else 1))
    if w["kind"] == "syrk":
        return e * (w["n"] * w["k"] + w["n"] * (w["n"] + 1) // 2 * (2 if w["beta"] != 0 else 1))
    if w["kind"] == "trsm":
        return e * (w["m"] * (w["m"] + 1) // 2 + 2 * w["m"] * w["n"])
    if w["kind"] == "strided":
        m, n, k, b = w["m"], w["n"], w["k"], w["batch"]
        return e * b * (m * k + k * n + m * n * (2 if w["beta"] != 0 else 1))
    oh = (w["height"] + 2 * w["pad"] - w["dil"] * (w["kh"] - 1) - 1) // w["stride"] + 1
    ow = (w["width"] + 2 * w["pad"] - w["dil"] * (w["kw"] - 1) - 1) // w["stride"] + 1
    return e * (w["batch"] * w["channels"] * w["height"] * w["width"] + w["num_kernels"] * w["channels"] * w["kh"] * w["kw"]
                + w["batch"] * w["num_kernels"] * oh * ow)


def config_of(name, w, **extra):
    """The `config` object both arms print: the workload's name and parameters."""
    return {"workload": name, **{k: v for k, v in w.items() if k not in ("kind", "bound")}, **extra}


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def traffic_from_profile(workload):
    """dram__bytes_read.sum + dram__bytes_write.sum per launch as recorded in the ncu summary of the workload."""
    name = PROFILE_OF.get(workload)
    if not name or not (ROOT / "profiles" / name).exists():
        return None
    m = re.search(r"`roofline\.traffic` for bench\.py:\s*([0-9.eE+]+)\s*bytes per launch",
                  (ROOT / "profiles" / name).read_text())
    return float(m.group(1)) if m else None


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []
        self.reader = None

    def start(self):
        """Starts nvidia-smi and returns once its first sample has arrived (several ranks starting it at once take a
        few hundred milliseconds), so that the samples that follow fall into the region being timed."""
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "10"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return

        def pump():
            for line in self.proc.stdout:
                self.lines.append((time.monotonic(), line))

        self.reader = threading.Thread(target=pump, daemon=True)
        self.reader.start()
        deadline = time.monotonic() + 5.0
        while not self.lines and time.monotonic() < deadline and self.proc.poll() is None:
            time.sleep(0.01)
        self.begin = time.monotonic()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.05)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        if self.reader is not None:
            self.reader.join(timeout=2)
        # the samples taken since start() returned; all of them when the region was shorter than one sampling period
        chosen = [line for stamp, line in self.lines if stamp >= self.begin] or [line for _, line in self.lines]
        sm, smax, reasons, power = [], [], set(), []
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in chosen:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
                power.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def fill_big(torch, count, dt, gen, device, dist_name="uniform1"):
    """Seeded values generated in slices: torch.rand materialises fp32 temporaries of the slice only."""
    out = torch.empty(count, device=device, dtype=dt)
    step_ = 1 << 28
    for s0 in range(0, count, step_):
        e0 = min(count, s0 + step_)
        if dist_name == "normal0.1":
            out[s0:e0] = (torch.randn(e0 - s0, generator=gen, device=device, dtype=torch.float32) * 0.1).to(dt)
        elif dt.is_complex:
            re = torch.rand(e0 - s0, generator=gen, device=device, dtype=torch.float32) * 2 - 1
            im = torch.rand(e0 - s0, generator=gen, device=device, dtype=torch.float32) * 2 - 1
            out[s0:e0] = torch.complex(re, im).to(dt)
        else:
            out[s0:e0] = (torch.rand(e0 - s0, generator=gen, device=device, dtype=torch.float32) * 2 - 1).to(dt)
    return out


def make_inputs(torch, w, device, seed, rows_scale=1):
    """Device tensors for one workload, generated on the device from a seed. rows_scale multiplies M (gemm only)."""
    g = torch.Generator(device=device).manual_seed(seed)
    dt = getattr(torch, TORCH_DT[w["precision"]])

    def fill(n):
        return fill_big(torch, n, dt, g, device, w.get("dist", "uniform1"))

    if w["kind"] == "syrk":
        n, k = w["n"], w["k"]
        return dict(a=fill(n * k), c=torch.full((n * n,), float("nan"), device=device, dtype=dt))
    if w["kind"] == "trsm":
        m, n = w["m"], w["n"]
        a = fill(m * m) * 0.01                      # small off-diagonal entries, unit-sized diagonal: well conditioned
        a.view(m, m).diagonal().add_(1.0)
        b = fill(m * n)
        return dict(a=a, b=b, b0=b.clone())
    if w["kind"] == "gemm":
        m, n, k = w["m"] * rows_scale, w["n"], w["k"]
        pad = w.get("ld_pad", 0)
        a_one, a_two = ((k, m) if w["ta"] == NO else (m, k)) if w["layout"] == ROW else ((m, k) if w["ta"] == NO else (k, m))
        b_one, b_two = ((n, k) if w["tb"] == NO else (k, n)) if w["layout"] == ROW else ((k, n) if w["tb"] == NO else (n, k))
        c_one, c_two = (n, m) if w["layout"] == ROW else (m, n)
        geo = dict(a_ld=a_one + pad, b_ld=b_one + pad, c_ld=c_one + pad)
        a = fill(geo["a_ld"] * a_two)
        b = fill(geo["b_ld"] * b_two)
        c = fill(geo["c_ld"] * c_two) if w["beta"] != 0 else torch.full((geo["c_ld"] * c_two,), float("nan"), device=device, dtype=dt)
        return dict(a=a, b=b, c=c, **geo)
    if w["kind"] == "sharded":
        from clblast_b200.multi_gpu import split_range
        world = int(os.environ.get("WORLD_SIZE", "1"))
        rank = int(os.environ.get("RANK", "0"))
        m, n, k = w["m"], w["n"], w["k"]
        j0, j1 = split_range(n, world, 256)[rank]
        n_local = j1 - j0
        # rank 0 owns A (other ranks receive it; their copy starts out poisoned); B's column block is per rank
        a = fill(m * k) if rank == 0 else torch.full((m * k,), float("nan"), device=device, dtype=dt)
        b = fill(k * n_local)
        c = torch.full((m * n_local,), float("nan"), device=device, dtype=dt)
        return dict(a=a, b=b, c=c, a_ld=m, b_ld=k, c_ld=m, n_local=n_local, j0=j0)
    if w["kind"] == "strided":
        m, n, k, bt = w["m"], w["n"], w["k"], w["batch"] * rows_scale
        return dict(a=fill(bt * m * k), b=fill(bt * k * n), c=fill(bt * m * n), batch=bt)
    bt = w["batch"] * rows_scale
    oh = (w["height"] + 2 * w["pad"] - w["dil"] * (w["kh"] - 1) - 1) // w["stride"] + 1
    ow = (w["width"] + 2 * w["pad"] - w["dil"] * (w["kw"] - 1) - 1) // w["stride"] + 1
    im = fill(bt * w["channels"] * w["height"] * w["width"])
    ker = (torch.randn(w["num_kernels"] * w["channels"] * w["kh"] * w["kw"], generator=g, device=device) * 0.05).to(dt)
    res = torch.full((bt * w["num_kernels"] * oh * ow,), float("nan"), device=device, dtype=dt)
    return dict(a=im, b=ker, c=res, batch=bt)


def launch(cb, w, t, stream, m_override=None):
    """One step of the workload on `stream` (None = the reference's host-synchronous semantics)."""
    if w["kind"] == "syrk":
        return cb.Syrk(w["layout"], 122, NO, w["n"], w["k"], w["alpha"], t["a"], 0, w["n"], w["beta"], t["c"], 0, w["n"],
                       stream=stream)
    if w["kind"] == "trsm":
        t["b"].copy_(t["b0"])     # the solve overwrites B: every step starts from the same right-hand side
        return cb.Trsm(w["layout"], 141, 122, NO, 131, w["m"], w["n"], w["alpha"], t["a"], 0, w["m"], t["b"], 0, w["m"],
                       stream=stream)
    if w["kind"] == "gemm":
        m = m_override or w["m"]
        return cb.Gemm(w["layout"], w["ta"], w["tb"], m, w["n"], w["k"], w["alpha"], t["a"], 0, t["a_ld"], t["b"], 0,
                       t["b_ld"], w["beta"], t["c"], 0, t["c_ld"], stream=stream)
    if w["kind"] == "sharded":
        if t["n_local"] == 0:
            return 0
        return cb.Gemm(w["layout"], w["ta"], w["tb"], w["m"], t["n_local"], w["k"], w["alpha"], t["a"], 0, t["a_ld"],
                       t["b"], 0, t["b_ld"], w["beta"], t["c"], 0, t["c_ld"], stream=stream)
    if w["kind"] == "strided":
        m, n, k = w["m"], w["n"], w["k"]
        return cb.GemmStridedBatched(w["layout"], w["ta"], w["tb"], m, n, k, w["alpha"], t["a"], 0, m, m * k, t["b"], 0,
                                     k, k * n, w["beta"], t["c"], 0, m, m * n, t["batch"], stream=stream)
    return cb.Convgemm(151, w["channels"], w["height"], w["width"], w["kh"], w["kw"], w["pad"], w["pad"], w["stride"],
                       w["stride"], w["dil"], w["dil"], w["num_kernels"], t["batch"], t["a"], 0, t["b"], 0, t["c"], 0,
                       stream=stream)


def time_steps(torch, fn, steps, warmup, dist=None, per_step=None):
    """Warm-up, then exactly `steps` calls bracketed by barrier + synchronize; returns the max-over-ranks ms of the
    whole region. With `per_step` (a list), an event after every call gives the individual step times too."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)] if per_step is not None else None
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    if marks:
        marks[0].record()
    for i in range(steps):
        fn()
        if marks:
            marks[i + 1].record()
    end.record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    ms = start.elapsed_time(end)
    if marks:
        per_step.extend(marks[i].elapsed_time(marks[i + 1]) for i in range(steps))
    if dist is not None:
        tms = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        ms = float(tms.item())
    return ms


def kernel_time(torch, fn, steps):
    """Device time of one launch of `fn` on the current stream: (best estimate ms, dict of statistics).

    Launches are timed one by one with CUDA events (median and minimum over `steps`, after 3 warm-up launches).
    Kernels shorter than the host's per-call cost are also replayed from a CUDA graph of 50 launches, so that the GPU,
    not the Python caller, sets the pace; the smaller of the two figures is the estimate."""
    each = []
    total = time_steps(torch, fn, steps, 3, None, per_step=each)
    stats = {"mean_ms": total / steps, "median_ms": statistics.median(each), "min_ms": min(each),
             "timing": "cuda events, back-to-back launches"}
    best = stats["median_ms"]
    if best < 0.2:
        try:
            reps = 50
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                fn()
                side.synchronize()
                with torch.cuda.graph(graph, stream=side):
                    for _ in range(reps):
                        fn()
            torch.cuda.synchronize()
            rounds = max(3, steps // 4)
            each_g = []
            time_steps(torch, graph.replay, rounds, 2, None, per_step=each_g)
            gms = statistics.median(each_g) / reps
            stats["graph_ms"] = gms
            if gms < best:
                best = gms
                stats["timing"] = f"cuda events around a CUDA graph of {reps} launches (median of {rounds} replays)"
        except Exception as exc:  # capture is an optimisation of the measurement only
            stats["timing"] += f" (graph capture unavailable: {type(exc).__name__})"
    return best, stats


def probe_peaks(torch, device):
    """Library GEMMs (cuBLAS through torch.matmul, 8192^3, best of 5) as roofline denominators for the precisions
    MEASURED_PEAKS.json has no entry for. A peak probe outside every timed region, not a product path."""
    n = 8192
    out = {}
    old = torch.backends.cuda.matmul.allow_tf32
    try:
        for name, dt, tf32 in (("fp32_tflops", torch.float32, False), ("tf32_tflops", torch.float32, True),
                               ("fp64_tflops", torch.float64, False), ("fp16_tflops", torch.float16, False)):
            torch.backends.cuda.matmul.allow_tf32 = tf32
            a = torch.randn(n, n, device=device, dtype=dt)
            b = torch.randn(n, n, device=device, dtype=dt)
            torch.matmul(a, b)
            torch.cuda.synchronize()
            best = float("inf")
            for _ in range(5):
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                torch.matmul(a, b)
                e.record()
                torch.cuda.synchronize()
                best = min(best, s.elapsed_time(e))
            out[name] = 2.0 * n ** 3 / (best * 1e-3) / 1e12
            del a, b
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    torch.cuda.empty_cache()
    out["how"] = "torch.matmul 8192^3, best of 5, CUDA events, measured in this run"
    out["nominal_ffma_tflops"] = 148 * 128 * 2 * 1.965e9 / 1e12
    return out


def roofline_of(w, kernel_name, kms, peaks, peak_kind, probed, flops):
    """The roofline object of one workload: algorithmic bytes or flops of one launch over its device time."""
    bound = w["bound"]
    if bound == "hbm":
        achieved = min_bytes_of(w) / (kms * 1e-3) / 1e9
        peak = float(peaks["hbm_gbs"])
        roof = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": None, "peak_source": f"{peak_kind} STREAM-style copy"}
    else:
        achieved = flops / (kms * 1e-3) / 1e12
        if bound == "tensor":
            peak = float(peaks["bf16_tflops"])
            src = f"{peak_kind} cuBLAS bf16 burst"
        elif bound == "fp32" and "tc_" in kernel_name:
            # error-compensated 3xTF32: three tensor-core products per fp32 product
            bound = "tensor"
            peak = (probed or {}).get("tf32_tflops", 756.0) / 3
            src = ("cuBLAS TF32 measured in this run / 3 tensor-core products per fp32 product" if probed else
                   "cuBLAS TF32 measured on this pool earlier (756 TFLOP/s) / 3")
        elif bound == "fp32":
            peak = (probed or {}).get("fp32_tflops", 64.0)
            src = "cuBLAS fp32 (TF32 off) measured in this run" if probed else "cuBLAS fp32 measured on this pool earlier"
        else:
            peak = (probed or {}).get("fp64_tflops", 35.5)
            src = "cuBLAS fp64 measured in this run" if probed else "cuBLAS fp64 measured on this pool earlier"
        roof = {"bound": bound, "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "traffic": None, "peak_source": src}
    roof["kernel"] = kernel_name
    roof["kernel_ms"] = kms
    roof["algorithmic_bytes"] = min_bytes_of(w)
    return roof


# ---- CPU legs (the only place the oracle is executed outside tests) ----------------------------------------

def cpu_sample(w, seconds_target=12.0):
    """Times the oracle port on a bounded sample of the workload. Returns (tflops, cores, description)."""
    cores = os.cpu_count() or 1
    # torchrun pins OMP_NUM_THREADS to 1 for its workers; the CPU baseline uses every host core, so the variable is
    # set before the OpenMP runtime inside the oracle library is loaded.
    os.environ["OMP_NUM_THREADS"] = str(cores)
    from oracle import cpu_oracle as oracle
    oracle.build()
    rng = np.random.default_rng(0)
    p = w["precision"]
    dt = oracle.NP_OF[p]

    def draw(count):
        if w.get("dist") == "normal0.1":
            return (rng.standard_normal(count) * 0.1).astype(dt)
        return rng.uniform(-1, 1, count).astype(dt)

    if w["kind"] in ("gemm", "sharded"):
        n, k = w["n"], w["k"]
        # a block of rows of C with the full N and K: same inner loops, bounded work
        rate_guess = {16: 3e9, 32: 30e9, 64: 15e9}[p] * max(1, cores // 8)
        rows = int(max(8, min(w["m"], seconds_target * rate_guess / (2.0 * n * k))))
        a = draw(rows * k)
        b = draw(n * k)
        c = np.zeros(rows * n, dtype=dt)
        # row-major NoTrans/Trans geometry for the headline; other GEMM workloads use the same sample geometry
        t0 = time.perf_counter()
        oracle.gemm(p, ROW, NO, YES, rows, n, k, w["alpha"], a, 0, k, b, 0, k, 0.0, c, 0, n)
        dtm = time.perf_counter() - t0
        return 2.0 * rows * n * k / dtm / 1e12, cores, f"{rows} of {w['m']} rows of C (full N={n}, K={k}), type-T reference order, {dtm:.1f} s"
    if w["kind"] == "strided":
        m, n, k = w["m"], w["n"], w["k"]
        nb = w["batch"]
        a = draw(nb * m * k)
        b = draw(nb * k * n)
        c = draw(nb * m * n)
        t0 = time.perf_counter()
        for i in range(nb):
            oracle.gemm(p, COL, NO, NO, m, n, k, 1.0, a, i * m * k, m, b, i * k * n, k, 1.0, c, i * m * n, m)
        dtm = time.perf_counter() - t0
        return 2.0 * nb * m * n * k / dtm / 1e12, cores, f"{nb} of {w['batch']} batches, {dtm:.1f} s"
    nb = min(w["batch"], 32)
    im = rng.uniform(-1, 1, nb * w["channels"] * w["height"] * w["width"]).astype(dt)
    ker = (rng.standard_normal(w["num_kernels"] * w["channels"] * w["kh"] * w["kw"]) * 0.05).astype(dt)
    oh, ow = oracle.conv_output_size(w["height"], w["width"], w["kh"], w["kw"], w["pad"], w["pad"], w["stride"],
                                     w["stride"], w["dil"], w["dil"])
    res = np.zeros(nb * w["num_kernels"] * oh * ow, dtype=dt)
    t0 = time.perf_counter()
    oracle.convgemm(p, 151, w["channels"], w["height"], w["width"], w["kh"], w["kw"], w["pad"], w["pad"], w["stride"],
                    w["stride"], w["dil"], w["dil"], w["num_kernels"], nb, im, 0, ker, 0, res, 0)
    dtm = time.perf_counter() - t0
    return flops_of(w) / w["batch"] * nb / dtm / 1e12, cores, f"{nb} of {w['batch']} images, {dtm:.1f} s"


def run_reference_arm(args, w, name):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals = []
    sample = ""
    cores = 1
    for i in range(args.warmup + args.steps):
        v, cores, sample = cpu_sample(w, seconds_target=3.0)
        if i >= args.warmup:
            vals.append(v)
    value = sum(vals) / len(vals)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    line = {"impl": "reference", "metric": "gemm_tflops", "value": value, "unit": "TFLOPS", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True,
            "scaling": "strong" if w["kind"] == "sharded" else "weak",
            "vs_baseline": None, "dtype": DTYPE_NAME[w["precision"]], "data": "synthetic",
            "config": gpu_config(name, w, world),
            "median": statistics.median(vals), "best": max(vals),
            "cpu_baseline": {"value": value, "unit": "TFLOPS", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def gpu_config(name, w, n_gpus):
    """`config` of both arms: identical for the same workload and GPU count."""
    return config_of(
        name, w,
        per_gpu=("one full copy of the workload per GPU; B re-sent from rank 0 every step, overlapped with the "
                 "previous step's GEMM") if n_gpus > 1 else "single GPU",
        l2=("inputs larger than L2 (no flush needed)" if min_bytes_of(w) > 126e6
            else "working set fits in L2; no flush between iterations"))


# ---- the reference's own CUDA build on the same GPU (separate process: it exports the same symbols) -----------

def reference_on_gpu(timeout_s=240):
    """Runs baseline/run_reference (built by baseline/build_reference.py where the reference tree was present) and
    returns its JSON, or a dict with the reason it is unavailable."""
    exe = ROOT / "baseline" / "_ref" / "run_reference"
    if not exe.exists():
        return {"unavailable": "baseline/_ref/run_reference has not been built (the reference tree was absent)"}
    try:
        res = subprocess.run([str(exe)], capture_output=True, text=True, timeout=timeout_s,
                             env={**os.environ, "LD_LIBRARY_PATH": f"{exe.parent}:{os.environ.get('LD_LIBRARY_PATH', '')}"})
    except subprocess.TimeoutExpired:
        return {"unavailable": f"the reference run did not finish within {timeout_s} s"}
    except OSError as exc:
        return {"unavailable": f"could not start the reference run: {exc}"}
    for ln in reversed(res.stdout.splitlines()):
        if ln.startswith("{"):
            try:
                out = json.loads(ln)
                if res.stderr.strip():
                    out["stderr_tail"] = res.stderr.strip()[-400:]
                return out
            except ValueError:
                break
    return {"unavailable": f"the reference run exited with {res.returncode}: {(res.stderr or res.stdout)[-300:]}"}


# ---- GPU arm ------------------------------------------------------------------------------------------------

def sharded_block(torch, cb, dist, device, names, steps=3):
    """The column-sharded problems at this number of GPUs (strong scaling): TFLOPS with and without re-sending A."""
    from clblast_b200.multi_gpu import CopyEngineFanout
    world = dist.get_world_size() if dist is not None else 1
    rank = dist.get_rank() if dist is not None else 0
    out = {}
    for name in names:
        w = WORKLOADS[name]
        entry = {}
        try:
            elem = ELEM[w["precision"]]
            free, _ = torch.cuda.mem_get_info()
            need = elem * (w["m"] * w["k"] + (w["k"] + w["m"]) * (-(-w["n"] // world))) + (4 << 30)
            if free < need:
                raise RuntimeError(f"needs {need >> 30} GiB of device memory, {free >> 30} GiB free")
            t = make_inputs(torch, w, device, seed=4321 + rank)
            stream = torch.cuda.current_stream()
            fan = None
            if world > 1:
                # A arrives from rank 0 in every step; one buffer, so a step is copy then GEMM
                fan = CopyEngineFanout(dist, [t["a"]], root=0)

            def plain():
                st = launch(cb, w, t, stream)
                if st != 0:
                    raise RuntimeError(f"library call failed with status {st}")

            def with_a():
                fan.step_begin(stream)
                plain()
                fan.step_end(stream)

            with_resend = None
            if fan is not None:   # first: it is what brings A to the other ranks at all
                ms_a = time_steps(torch, with_a, steps, 1, dist) / steps
                with_resend = {"tflops": flops_of(w) / (ms_a * 1e-3) / 1e12, "ms_per_step": ms_a,
                               "how": "binomial tree of copy-engine copies from rank 0, then the GEMM",
                               "bytes": elem * w["m"] * w["k"]}
            ms_plain = time_steps(torch, plain, steps, 1, dist) / steps
            entry = {"tflops": flops_of(w) / (ms_plain * 1e-3) / 1e12, "ms_per_step": ms_plain,
                     "n_local": t["n_local"], "kernel": cb.last_kernel(), "steps": steps,
                     "a_resend": "none (single GPU)" if world == 1 else "excluded"}
            if with_resend is not None:
                entry["with_a_resend"] = with_resend
            entry["max_error"] = sharded_error(torch, w, t)
            if dist is not None:
                e = torch.tensor([entry["max_error"]], device="cuda", dtype=torch.float64)
                dist.all_reduce(e, op=dist.ReduceOp.MAX)
                entry["max_error"] = float(e.item())
            entry["error_metric"] = "max |x - r| / sum_k |a||b| over 256 sampled entries per rank, r an fp64 dot product"
            if fan is not None:
                fan.close()
            del t
        except Exception as exc:  # a sharded entry must never take the headline down
            entry = {"error": f"{type(exc).__name__}: {exc}"}
        torch.cuda.empty_cache()
        if dist is not None:
            dist.barrier()
        out[name] = entry
    return out


def sharded_error(torch, w, t):
    """Sampled check of this rank's column block on the device in fp64 (16 rows x 16 columns)."""
    m, k, nl = w["m"], w["k"], t["n_local"]
    if nl == 0:
        return 0.0
    g = torch.Generator(device="cpu").manual_seed(7)
    rows = torch.cat([torch.tensor([0, m - 1]), torch.randint(0, m, (14,), generator=g)]).cuda()
    cols = torch.cat([torch.tensor([0, nl - 1]), torch.randint(0, nl, (14,), generator=g)]).cuda()
    kk = torch.arange(k, device="cuda", dtype=torch.int64)
    a_rows = t["a"][(rows[:, None] + kk[None, :] * m).reshape(-1)].view(16, k).double()
    b_cols = t["b"][(cols[:, None] * k + kk[None, :]).reshape(-1)].view(16, k).double()
    want = a_rows @ b_cols.T
    mag = a_rows.abs() @ b_cols.abs().T
    got = t["c"][(cols[None, :] * m + rows[:, None]).reshape(-1)].view(16, 16).double()
    return float(((got - want).abs() / mag).max().item())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="hgemm_8192", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=("b200", "reference"))
    ap.add_argument("--no-sweep", action="store_true", help="skip the per-config sweep added at N=1")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-sharded", action="store_true", help="skip the column-sharded problems")
    ap.add_argument("--no-reference-gpu", action="store_true", help="skip the reference's CUDA build on this GPU")
    ap.add_argument("--bcast", default="ce", choices=("ce", "nccl"),
                    help="how B reaches the ranks at N>1: copy-engine tree (default) or NCCL broadcast")
    ap.add_argument("--sm-budget", type=int, default=-1,
                    help="SMs the persistent GEMM kernels may use; default: all, except 132 of 148 at N>1 with "
                         "--bcast nccl so that the overlapped collective has SMs to run on")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg (profiling runs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    w = WORKLOADS[args.workload]

    if args.impl == "reference":
        run_reference_arm(args, w, args.workload)
        return

    import torch
    import clblast_b200 as cb
    cb.lib()  # fail loudly when the native library is missing: there is no fallback
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200); nothing is computed on the host")

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as tdist
        tdist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist = tdist
    if args.gpus != world and rank == 0:
        print(f"note: --gpus {args.gpus} but WORLD_SIZE is {world}; using {world}", file=sys.stderr)
    n_gpus = world
    replicate_b = dist is not None and w["kind"] == "gemm"
    use_nccl = replicate_b and args.bcast == "nccl"
    sm_budget = args.sm_budget if args.sm_budget >= 0 else (132 if use_nccl else 0)
    cb.set_sm_budget(sm_budget)
    device = torch.device("cuda", local_rank)
    peaks, peak_kind = load_peaks()

    # Per-rank problem: every rank owns one full copy of the workload's M rows (weak scaling); for the GEMM
    # workloads rank 0's B is the one everybody uses and is re-sent inside every step.
    t = make_inputs(torch, w, device, seed=1234 + rank)
    stream = torch.cuda.current_stream()

    # With N > 1 the operand every rank needs whole (B here) leaves rank 0 again in every step, into a second buffer
    # while the GEMM of the previous step runs, so a step costs max(transfer, GEMM) in steady state; every step still
    # contains one transfer to every rank and one GEMM per rank.
    bcast = {"bufs": None, "cur": 0, "work": None, "fan": None}
    bcast_how = None
    if replicate_b:
        # Three ring slots for the copy-engine tree: the copy of step s + 3 into a slot may start as soon as the GEMM of
        # step s is done, which leaves it two GEMMs' time to cross up to three hops while copies share HBM and NVLink
        # with the running GEMMs (with two slots and eight ranks the leaves waited: 0.87 ms per step against 0.77).
        bcast["bufs"] = [t["b"]] + [torch.empty_like(t["b"]) for _ in range(1 if use_nccl else 2)]
        dist.broadcast(bcast["bufs"][0], src=0)     # set-up, outside every timed region
        for extra in bcast["bufs"][1:]:
            extra.copy_(bcast["bufs"][0])
        torch.cuda.synchronize()
        if not use_nccl:
            try:
                from clblast_b200.multi_gpu import CopyEngineFanout
                bcast["fan"] = CopyEngineFanout(dist, bcast["bufs"], root=0)
                bcast_how = "binomial tree of cudaMemcpyAsync peer copies (copy engines), three ring slots"
            except Exception as exc:
                flag = torch.tensor([1], device="cuda")
                print(f"note: copy-engine fan-out unavailable on rank {rank} ({exc}); falling back to NCCL", file=sys.stderr)
            else:
                flag = torch.tensor([0], device="cuda")
            dist.all_reduce(flag)
            if int(flag.item()) != 0:   # every rank takes the same path
                bcast["fan"] = None
                use_nccl = True
                sm_budget = args.sm_budget if args.sm_budget >= 0 else 132
                cb.set_sm_budget(sm_budget)
        if use_nccl:
            bcast_how = "ncclBroadcast on NCCL's stream, double buffered"

    def step():
        if bcast["fan"] is not None:
            t["b"] = bcast["fan"].step_begin(stream)
        elif bcast["bufs"] is not None:
            if bcast["work"] is not None:
                bcast["work"].wait()          # this step's B has arrived (stream-level wait, no host block)
                bcast["cur"] ^= 1
            t["b"] = bcast["bufs"][bcast["cur"]]
            bcast["work"] = dist.broadcast(bcast["bufs"][bcast["cur"] ^ 1], src=0, async_op=True)
        st = launch(cb, w, t, stream)
        if st != 0:
            raise RuntimeError(f"library call failed with status {st}")
        if bcast["fan"] is not None:
            bcast["fan"].step_end(stream)

    sampler = ClockSampler(local_rank)
    sampler.start()
    step()
    torch.cuda.synchronize()
    kernel_name = cb.last_kernel()

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    launches_before = cb.launch_count()
    each_step = []
    ms = time_steps(torch, step, args.steps, 0, dist, per_step=each_step)
    launches = cb.launch_count() - launches_before
    clocks = sampler.stop()
    if bcast["work"] is not None:
        bcast["work"].wait()
    torch.cuda.synchronize()
    if bcast["bufs"] is not None:
        t["b"] = bcast["bufs"][0]
    st_code, st_words = cb.tensor_core_status()
    if st_code != 0:
        raise RuntimeError(f"a tensor-core kernel reported an expired wait: {st_words}")

    # a sharded workload is ONE problem split over the ranks; every other workload is one full copy per rank
    total_flops = flops_of(w) * (1 if w["kind"] == "sharded" else n_gpus)
    ms_per_step = ms / args.steps
    value = total_flops / (ms_per_step * 1e-3) / 1e12

    # Library GEMMs as denominators for fp32 / tf32 / fp64 (rank 0 of a single-GPU run; elsewhere the earlier figures)
    probed = probe_peaks(torch, device) if (rank == 0 and n_gpus == 1) else None

    # Dominant kernel alone (no transfer), CUDA events on the launching stream: the roofline numerator.
    cb.set_sm_budget(0)  # the kernel alone may use every SM

    def kernel_only():
        launch(cb, w, t, torch.cuda.current_stream())
    kms, kstats = kernel_time(torch, kernel_only, args.steps)
    # the kernel of a sharded workload computes this rank's column block only
    kernel_flops = flops_of(w) * (t["n_local"] / w["n"] if w["kind"] == "sharded" else 1)
    roof = roofline_of(w, kernel_name, kms, peaks, peak_kind, probed, kernel_flops)
    roof.update(kstats)
    roof["traffic"] = traffic_from_profile(args.workload)
    if roof["traffic"] is not None:
        roof["traffic_source"] = f"profiles/{PROFILE_OF[args.workload]}"

    # The same step under sustained load (about 1.5 s back to back): on a 1 kW part a dense tensor kernel runs into
    # the power cap, so this is reported next to the burst number, with the clocks seen during it.
    sustained = None
    if roof["bound"] == "tensor" and w["bound"] == "tensor" and rank == 0 and n_gpus == 1:
        reps = max(args.steps, int(1500.0 / max(kms, 1e-3)))
        s2 = ClockSampler(local_rank)
        s2.start()
        sms = time_steps(torch, kernel_only, reps, 3, None) / reps
        sc = s2.stop()
        sustained = {"value": flops_of(w) / (sms * 1e-3) / 1e12, "unit": "TFLOPS", "launches": reps, "clocks": sc,
                     "peak": peaks.get("bf16_tflops_sustained"), "peak_source": f"{peak_kind} cuBLAS bf16 sustained"}
        if sustained["peak"]:
            sustained["frac"] = sustained["value"] / float(sustained["peak"])

    cb.set_sm_budget(sm_budget)
    # End to end through the API with pinned host buffers. Every rank loads all of its inputs (B included) from its
    # own pinned memory, so no rank waits for another one's host copy.
    host = {}
    h2d = d2h = 0
    needs_c_in = w.get("beta", 0.0) != 0
    if not args.no_e2e:
        host = {k: torch.empty(t[k].shape, dtype=t[k].dtype).pin_memory() for k in ("a", "b", "c")}
        for k in ("a", "b", "c"):
            host[k].copy_(t[k])
        h2d = host["a"].numel() * host["a"].element_size() + host["b"].numel() * host["b"].element_size()
        if needs_c_in:
            h2d += host["c"].numel() * host["c"].element_size()
        d2h = host["c"].numel() * host["c"].element_size()

    def e2e_step_simple():
        t["a"].copy_(host["a"], non_blocking=True)
        t["b"].copy_(host["b"], non_blocking=True)
        if needs_c_in:
            t["c"].copy_(host["c"], non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the library's private stream does not order against ours
        st = launch(cb, w, t, None)
        if st != 0:
            raise RuntimeError(f"library call failed with status {st}")
        host["c"].copy_(t["c"], non_blocking=True)
        torch.cuda.current_stream().synchronize()

    # Row-major GEMMs whose A is not transposed are streamed in row blocks: while block i is multiplied (one library
    # call per block, through the offset arguments of the API), block i+1 of A travels host->device and block i-1
    # of C device->host, so the PCIe link is busy in both directions instead of idling during the product.
    pipelined = (not args.no_e2e and w["kind"] == "gemm" and w["layout"] == ROW and w["ta"] == NO and w["m"] % 8 == 0)
    if pipelined:
        s_in, s_mm, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        blocks = 8
        rows = w["m"] // blocks

    def e2e_step_pipelined():
        start = torch.cuda.Event()
        start.record()
        for s_ in (s_in, s_mm, s_out):
            s_.wait_event(start)
        with torch.cuda.stream(s_in):
            t["b"].copy_(host["b"], non_blocking=True)
        for i in range(blocks):
            a0, a1 = i * rows * t["a_ld"], (i + 1) * rows * t["a_ld"]
            c0, c1 = i * rows * t["c_ld"], (i + 1) * rows * t["c_ld"]
            with torch.cuda.stream(s_in):
                t["a"][a0:a1].copy_(host["a"][a0:a1], non_blocking=True)
                if needs_c_in:
                    t["c"][c0:c1].copy_(host["c"][c0:c1], non_blocking=True)
                ready = torch.cuda.Event()
                ready.record()
            s_mm.wait_event(ready)
            st = cb.Gemm(w["layout"], w["ta"], w["tb"], rows, w["n"], w["k"], w["alpha"], t["a"], a0, t["a_ld"], t["b"], 0,
                         t["b_ld"], w["beta"], t["c"], c0, t["c_ld"], stream=s_mm)
            if st != 0:
                raise RuntimeError(f"library call failed with status {st}")
            with torch.cuda.stream(s_mm):
                done = torch.cuda.Event()
                done.record()
            s_out.wait_event(done)
            with torch.cuda.stream(s_out):
                host["c"][c0:c1].copy_(t["c"][c0:c1], non_blocking=True)
        for s_ in (s_in, s_mm, s_out):
            torch.cuda.current_stream().wait_stream(s_)
        torch.cuda.current_stream().synchronize()  # the result is in host memory when the step ends

    e2e_step = e2e_step_pipelined if pipelined else e2e_step_simple

    e2e_steps = max(3, min(args.steps, 10))
    if args.no_e2e:
        e2e_ms, e2e_value = None, None
    else:
        e2e_ms = time_steps(torch, e2e_step, e2e_steps, 2, dist) / e2e_steps
        e2e_value = total_flops / (e2e_ms * 1e-3) / 1e12
        host.clear()

    cfg = gpu_config(args.workload, w, n_gpus)
    line = {
        "metric": "gemm_tflops", "value": value, "unit": "TFLOPS", "n_gpus": n_gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        # one problem split over the ranks keeps the total work fixed; every other workload is one copy per rank
        "scaling": "strong" if w["kind"] == "sharded" else "weak",
        "vs_baseline": None, "dtype": DTYPE_NAME[w["precision"]], "data": "synthetic",
        "config": cfg,
        "transport": {"sm_budget": sm_budget or "all", "b_resend": bcast_how},
        "step_ms": {"median": statistics.median(each_step), "min": min(each_step), "of": "rank 0's steps"},
        "roofline": roof,
        "e2e": {"value": e2e_value, "unit": "TFLOPS", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms,
                "how": "8 row blocks streamed: H2D of block i+1 and D2H of block i-1 overlap the product of block i"
                if pipelined else "copy in, one host-synchronous call, copy out"},
        "gpu_launches": int(launches),
        "clocks": clocks,
    }
    if sustained is not None:
        line["sustained"] = sustained
    if probed is not None:
        line["peaks"] = probed

    if bcast["fan"] is not None:
        bcast["fan"].close()
    del t
    bcast["bufs"] = None
    torch.cuda.empty_cache()
    cb.set_sm_budget(0)

    if rank == 0 and n_gpus == 1 and not args.no_sweep:
        sweep = {}
        for name, ww in WORKLOADS.items():
            if name == args.workload or ww["kind"] == "sharded":
                continue  # the sharded shapes take seconds per launch: they have their own block below
            try:
                # A working set that fits in L2 (126 MB) is rotated: consecutive launches use different copies of the
                # inputs, more than twice the L2 in total, so no launch finds its operands cached by the previous ones.
                copies = 1 if min_bytes_of(ww) > 126e6 else int(2 * 126e6 // min_bytes_of(ww)) + 1
                sets = [make_inputs(torch, ww, device, seed=99 + i) for i in range(copies)]
                turn = [0]

                def fn():
                    tt = sets[turn[0] % copies]
                    turn[0] += 1
                    return launch(cb, ww, tt, torch.cuda.current_stream())

                fn()
                torch.cuda.synchronize()
                kname = cb.last_kernel()
                ms_w, st_w = kernel_time(torch, fn, 10)
                entry = {"tflops": flops_of(ww) / (ms_w * 1e-3) / 1e12, "ms": ms_w,
                         "gbs": min_bytes_of(ww) / (ms_w * 1e-3) / 1e9, "kernel": kname,
                         "host_paced_ms": st_w["median_ms"], "min_ms": st_w["min_ms"],
                         "roofline": roofline_of(ww, kname, ms_w, peaks, peak_kind, probed, flops_of(ww)),
                         "l2": "inputs larger than L2" if copies == 1 else
                               f"launches rotate through {copies} copies of the inputs ({copies * min_bytes_of(ww) / 1e6:.0f} MB)"}
                entry["roofline"]["timing"] = st_w["timing"]
                sweep[name] = entry
                del sets
                torch.cuda.empty_cache()
            except Exception as exc:  # a sweep entry must never take the headline down
                sweep[name] = {"error": str(exc)}
        line["sweep"] = sweep

        # Wall clock around the public host-synchronous call (what a clblast::Gemm caller sees), as the reference's
        # own client measures (test/performance/client.cpp:419-468): minimum and median of 20 calls.
        sync_api = {}
        for name in ("sgemm_1024", "batched_32"):
            ww = WORKLOADS[name]
            try:
                tt = make_inputs(torch, ww, device, seed=99)
                torch.cuda.synchronize()
                for _ in range(3):
                    launch(cb, ww, tt, None)
                walls = []
                for _ in range(20):
                    t0 = time.perf_counter()
                    st = launch(cb, ww, tt, None)
                    walls.append((time.perf_counter() - t0) * 1e3)
                    if st != 0:
                        raise RuntimeError(f"status {st}")
                sync_api[name] = {"min_ms": min(walls), "median_ms": statistics.median(walls),
                                  "kernel_ms": sweep.get(name, {}).get("ms"), "calls": 20,
                                  "tflops_at_min": flops_of(ww) / (min(walls) * 1e-3) / 1e12}
                del tt
            except Exception as exc:
                sync_api[name] = {"error": str(exc)}
        torch.cuda.empty_cache()
        line["sync_api"] = sync_api

    if not args.no_sharded and w["kind"] != "sharded":
        block = sharded_block(torch, cb, dist, device, SHARDED_IN_EVERY_RUN)
        if rank == 0:
            line["sharded"] = block

    if rank == 0 and n_gpus == 1 and not args.no_reference_gpu:
        line["reference_b200"] = reference_on_gpu()

    if rank == 0 and n_gpus == 1 and not args.no_cpu:
        v, cores, sample = cpu_sample(w)
        line["cpu_baseline"] = {"value": v, "unit": "TFLOPS", "cores": cores, "kind": "port", "sample": sample}
    elif rank == 0:
        line["cpu_baseline"] = None

    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
