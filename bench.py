#!/usr/bin/env python
"""Benchmark of the CUDA backend on the five benchmark graphs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1..c5] [--impl reference]

Plain ``python bench.py`` (one GPU): workload c2, matmul 4096^3 + relu; one step =
one run of the compiled graph ("weak": the work per GPU is the whole graph).
Launched by torch.distributed.run (any world size, 1 included): workload c5, the
row-sharded 65536x8192x8192 matmul; one step = every rank computes its row block and
the blocks are exchanged; the total work is fixed ("strong"), so the values at
1, 2, 4 and 8 ranks are one curve.  By default the exchange of a step (peer-to-peer
copies, then a barrier) runs on a second stream while the next step's product is
computed; every step's exchange has completed when the timed region ends.  Prints
ONE JSON line on rank 0.

  value     graph throughput with inputs resident in device memory
  e2e       the same through host buffers: pinned host -> device copies of the
            inputs and a device -> host copy of the result inside the timed region
  roofline  the dominant kernel's achieved rate against the measured peak
  other_configs   the remaining graphs and the standalone bandwidth kernels, device-resident
  cpu_baseline / --impl reference
            the CPU loop-nest restatement of the reference's MLIR llvmir lowering
            (oracle/cpu_loopnest.c) on all host cores, its tile sizes tuned first with
            this repository's exploration driver
"""

from __future__ import annotations

import argparse
import importlib.util
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

L2_BYTES = 126 * 1024 * 1024
# DRAM bytes per launch of the dominant kernel from one ncu capture each
# (dram__bytes_read.sum + dram__bytes_write.sum, see profiles/); None = not captured.
NCU_TRAFFIC = {"c1": None, "c2": 327.6e6, "c3": 25.9e6, "c4": None, "c4a": 488.1e6, "c5": None,
               "pad512": None, "relu512": None}


def measured_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "source": "MEASURED_PEAKS.json (of measured)"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "recipe fallback (of fallback)"}


def under_torchrun() -> bool:
    return "TORCHELASTIC_RUN_ID" in os.environ or "LOCAL_RANK" in os.environ


# --------------------------------------------------------------------------- #
# clocks sampling
# --------------------------------------------------------------------------- #
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int) -> None:
        self.gpu_index = gpu_index
        self.proc = None
        self.lines: list[str] = []

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self) -> None:
        assert self.proc is not None and self.proc.stdout is not None
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm),
                "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- #
# CPU baseline (the reference arm)
# --------------------------------------------------------------------------- #
def cpu_sample(workload: str) -> tuple:
    """(sample graph, inputs, description, fraction of the full workload) of the bounded CPU
    sample: the full graph, except for c5 where rows 0..1024 of A stand for all 65536."""
    from xtc_b200 import configs

    if workload == "c5":
        rows = 1024  # 1/64 of the rows; the time scales linearly with the rows
        cfg = configs.build("c5", rows=rows)
        return cfg, configs.input_rows("c5", 0, rows), f"rows 0..{rows} of A (1/64 of the work), all of B", rows / 65536
    return configs.build(workload), configs.inputs(workload), "the full workload", 1.0


def blas_ceiling(workload: str, ins: list, flops: float, frac: float) -> dict | None:
    """NumPy / OpenBLAS time of the same sample (matmul graphs only): a sanity ceiling for
    the loop nests, not the reference's own code generator."""
    if workload not in ("c1", "c2", "c4", "c5"):
        return None
    a, b = ins

    def run() -> None:
        lhs = a.T if workload == "c4" else a
        out = lhs @ b
        if workload == "c2":
            np.maximum(out, 0, out=out)

    run()
    times = []
    for _ in range(3):
        t0 = time.perf_counter()
        run()
        times.append(time.perf_counter() - t0)
    return {"value": flops * frac / min(times) / 1e12, "unit": "TFLOP/s",
            "what": "NumPy/OpenBLAS sgemm on the same sample and cores (its own thread count)"}


def time_cpu(workload: str, steps: int, warmup: int, trials: int = 16) -> dict:
    """Tunes the CPU loop nests on this host with the exploration driver (random search over
    two-level tile sizes and register tiles), then times the best sample on all host cores.
    Returns the cpu_baseline object plus `seconds_per_sample`."""
    from oracle import cpu_backend as cpb
    from oracle import cpu_baseline as cb

    cfg, ins, desc, frac = cpu_sample(workload)
    full_flops = cfg.flops / frac if cfg.flops else 0.0
    sample, tuned = None, "no contraction to tune"
    if cfg.flops:
        t0 = time.perf_counter()
        sample, best_sec, n = cpb.tune(cfg.graph, trials=trials, inputs=ins)
        names = cpb.StrategyCpuTile(cfg.graph).sample_names
        tuned = (f"best of {n} random samples of the two-level tiled, packed, register-blocked nest: "
                 f"{dict(zip(names, sample))} (tuning took {time.perf_counter() - t0:.1f} s, untimed)")
    name = "c5" if workload == "c5" else workload
    for _ in range(max(warmup, 1)):
        cb.run_config(name, ins, sample)
    times = []
    for _ in range(max(steps, 1)):
        t0 = time.perf_counter()
        cb.run_config(name, ins, sample)
        times.append(time.perf_counter() - t0)
    t = min(times)
    if cfg.flops:
        value, unit = full_flops * frac / t / 1e12, "TFLOP/s"
    else:
        value, unit = cfg.bytes / t / 1e9, "GB/s"
    out = {"value": value, "unit": unit, "cores": cb.threads(), "kind": "port",
           "sample": f"{desc}; {tuned}; best of {len(times)} timed runs, {t * 1e3:.1f} ms each",
           "seconds_per_sample": t}
    if cfg.flops:
        peak = cb.peak_fma() * 2 / 1e12
        out["host_fma_peak_tflops"] = peak
        out["frac_of_host_fma_peak"] = value / peak
        out["blas_ceiling"] = blas_ceiling(workload, ins, full_flops, frac)
    return out


def mlir_toolchain_present() -> bool:
    """Whether the reference's own code generator could run here (MLIR python bindings and
    xdsl importable).  It never is on this image; the line says so instead of assuming it."""
    return all(importlib.util.find_spec(m) is not None for m in ("mlir", "xdsl"))


def run_reference(args, rank: int, world: int) -> None:
    if rank != 0:
        return
    workload = args.workload or default_workload()
    steps = min(args.steps, 5)
    warm = min(args.warmup, 1)
    base = time_cpu(workload, steps, warm)
    t = base.pop("seconds_per_sample")
    line = {
        "impl": "reference", "metric": "graph_throughput", "value": base["value"],
        "unit": base["unit"], "n_gpus": world, "steps": steps, "warmup": warm,
        "ms_per_step": t * 1e3, "higher_is_better": True,
        "scaling": "strong" if under_torchrun() else "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": workload_name(workload)},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": base["unit"], "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "mlir_toolchain_present": mlir_toolchain_present(),
        "note": ("the reference's MLIR llvmir backend cannot be built on this box (no MLIR/LLVM "
                 "toolchain); this is its loop nest restated in C with the tile sizes tuned on "
                 "this host, OpenMP over the host cores"),
    }
    print(json.dumps(line), flush=True)


def default_workload() -> str:
    """c2 for a plain one-GPU run; c5 when launched by torch.distributed.run, at every world
    size, so that the 1/2/4/8-rank values are the same work."""
    return "c5" if under_torchrun() else "c2"


def workload_name(w: str) -> str:
    return {
        "c1": "c1: matmul 512x1024x256 f32",
        "c2": "c2: matmul 4096^3 + relu f32 (configs[1])",
        "c3": "c3: pad + conv2d 3x3 + relu, NHWC 32x56x56x64 -> 64 f32",
        "c4": "c4: transpose 8192^2 + matmul 8192x8192x1024 f32",
        "c4a": "c4a: transpose 8192^2 f32 alone",
        "c5": "c5: row-sharded matmul 65536x8192x8192 f32 + all-gather",
        "relu512": "standalone relu, 512 MiB tensor",
        "pad512": "standalone pad of H and W by 1, 512 MiB tensor",
    }[w]


# --------------------------------------------------------------------------- #
# our arm
# --------------------------------------------------------------------------- #
def pinned_like(dev, arr: np.ndarray) -> np.ndarray:
    """A pinned host copy of `arr` (cudaMallocHost through the C ABI)."""
    import ctypes

    from xtc_b200 import capi

    ptr = ctypes.c_void_p()
    capi.check(dev.lib.xtc_cuda_host_alloc(ctypes.byref(ptr), max(arr.nbytes, 4)))
    buf = (ctypes.c_float * max(arr.size, 1)).from_address(ptr.value)
    out = np.frombuffer(buf, dtype=np.float32, count=arr.size).reshape(arr.shape)
    np.copyto(out, arr)
    return out


def time_device_steps(torch, fn, steps: int, warmup: int, barrier=None, many=None):
    """W warm-up calls, then K calls bracketed by synchronize (+ barrier); returns
    (total seconds, list of average seconds per call of each timed segment), both
    from events on the current stream.  `many(first, count)`, when given, issues the
    steps first .. first + count - 1 from one host call (xtc_cuda_plan_run_sets): a step
    of a few microseconds is shorter than a call from Python."""
    if many is not None:
        many(0, warmup)
    else:
        for i in range(warmup):
            fn(i)
    torch.cuda.synchronize()
    if barrier:
        barrier()
    # An event between two launches costs a few microseconds of stream time, which is
    # not negligible next to a 10-30 us step: record one every `stride` steps (at most
    # 16 segments, 4 for short runs) and report each segment's average step time.
    stride = max(1, -(-steps // (16 if steps > 64 else 4)))
    marks = list(range(0, steps, stride)) + [steps]
    evs = [torch.cuda.Event(enable_timing=True) for _ in marks]
    torch.cuda.synchronize()
    evs[0].record()
    nxt = 1
    if many is not None:
        for j in range(len(marks) - 1):
            many(warmup + marks[j], marks[j + 1] - marks[j])
            evs[j + 1].record()
    else:
        for i in range(steps):
            fn(warmup + i)
            if i + 1 == marks[nxt]:
                evs[nxt].record()
                nxt += 1
    torch.cuda.synchronize()
    if barrier:
        barrier()
    per = [evs[j].elapsed_time(evs[j + 1]) * 1e-3 / (marks[j + 1] - marks[j])
           for j in range(len(marks) - 1)]
    return evs[0].elapsed_time(evs[-1]) * 1e-3, per


def bench_graph_device(torch, dev, name: str, steps: int, warmup: int, precision="tf32",
                       fuse_transpose=None, device_inputs=None, rows=None):
    """Device-resident throughput of one configuration on the current GPU."""
    from xtc_b200 import configs
    from xtc_b200.backends.cuda.module import PlanHandle

    cfg = configs.build(name, rows=rows) if rows else configs.build(name)
    module = configs.compile_config(cfg, precision=precision, fuse_transpose=fuse_transpose)
    plan = module.plan
    handle = PlanHandle(plan, dev)
    set_bytes = sum(plan.slot_bytes[: plan.n_inputs + plan.n_outputs])
    n_sets = int(min(max(2, math.ceil(3 * L2_BYTES / set_bytes)), 64))
    if set_bytes * n_sets > 40e9:
        n_sets = 2
    if device_inputs is None:
        host = configs.inputs(name)
        device_inputs = [torch.from_numpy(h).cuda() for h in host]
        del host
    sets = []
    for s in range(n_sets):
        ins = device_inputs if s == 0 else [t.clone() for t in device_inputs]
        out = torch.empty(cfg.output_shape, dtype=torch.float32, device="cuda")
        sets.append(([t.data_ptr() for t in ins] + [out.data_ptr()], ins, out))
    stream = torch.cuda.current_stream().cuda_stream

    table = handle.pointer_sets([s[0] for s in sets])

    def step(i: int) -> None:
        handle.run(sets[i % n_sets][0], stream)

    def many(first: int, count: int) -> None:
        handle.run_sets(table, first, count, stream)

    # every buffer set is visited once before timing (first visits record the CUDA graph)
    total, per = time_device_steps(torch, step, steps, max(warmup, n_sets), many=many)
    assert dev.status() == 0, "a kernel reported a bounded-wait timeout"
    info = {"cfg": cfg, "plan": plan, "seconds": total / steps, "per_step": per,
            "n_sets": n_sets, "set_bytes": set_bytes, "handle": handle, "sets": sets, "step": step,
            "many": many}
    return info


def measure_e2e(torch, dev, handle, cfg, workload: str, steps: int) -> dict:
    """The same steps through host buffers: every step copies its inputs from pinned
    host memory to the device and its result back.  Returns seconds per step of the
    pipelined executor and of the synchronous call, and the bytes moved per step."""
    from xtc_b200 import configs

    host_ins = [pinned_like(dev, h) for h in configs.inputs(workload)]
    host_out = pinned_like(dev, np.zeros(cfg.output_shape, np.float32))
    e2e_steps = max(3, min(steps, 20))
    for _ in range(2):
        handle.run_host(host_ins + [host_out])
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        handle.run_host(host_ins + [host_out])  # H2D inputs, run, D2H result, synchronise
    e2e_sync_sec = (time.perf_counter() - t0) / e2e_steps
    # the same steps through the pipelined executor: every step still copies all of its
    # inputs in and its result out, but step i+1's input copy and step i-1's output copy
    # overlap step i's kernels
    pipe = handle.pipeline(depth=3)
    host_outs = [host_out] + [pinned_like(dev, host_out) for _ in range(2)]
    for i in range(3):
        pipe.submit(host_ins + [host_outs[i % 3]])
    pipe.wait()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        pipe.submit(host_ins + [host_outs[i % 3]])
    pipe.wait()
    e2e_sec = (time.perf_counter() - t0) / e2e_steps
    pipe.close()
    h2d = int(sum(h.nbytes for h in host_ins))
    d2h = int(host_out.nbytes)

    return {"sec": e2e_sec, "sync_sec": e2e_sync_sec, "h2d": h2d, "d2h": d2h, "steps": e2e_steps}


def tf32_denominator(peaks: dict, sustained: bool) -> tuple[float, str]:
    """TF32 tensor peak used as the roofline denominator: half the measured dense bf16
    figure (kind::tf32 issues at half the bf16 rate; the driver-written file has no TF32
    entry), burst for a kernel timed alone, sustained for a seconds-long loop."""
    bf16 = peaks["bf16_tflops_sustained"] if sustained else peaks["bf16_tflops"]
    return bf16 / 2.0, (peaks["source"] + ": dense bf16 / 2 for TF32 ("
                        + ("sustained" if sustained else "burst") + ")")


def roofline_of(cfg, seconds: float, peaks: dict, workload: str, sustained: bool,
                precision: str = "tf32") -> dict:
    if cfg.bound == "hbm":
        achieved = cfg.bytes / seconds / 1e9
        return {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "traffic": NCU_TRAFFIC.get(workload),
                "peak_source": peaks["source"]}
    peak, source = tf32_denominator(peaks, sustained)
    if precision == "3xtf32":
        peak, source = peak / 3.0, source + " / 3 products per FMA"
    achieved = cfg.flops / seconds / 1e12
    return {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
            "frac": achieved / peak, "traffic": NCU_TRAFFIC.get(workload), "peak_source": source}


NVLINK_PEER_GBS = 770.0  # measured peer copy bandwidth per direction per GPU on this pool


def fused_roofline(flops_per_rank: float, exchange_bytes_per_rank: float, seconds: float,
                   peaks: dict) -> dict:
    """Roofline of a kernel that computes and exchanges at once: the target time is the
    slower of (FLOPs / measured TF32 GEMM peak) and (bytes each GPU must send over NVLink /
    measured link bandwidth); `frac` = target / measured."""
    compute = flops_per_rank / (peaks["bf16_tflops_sustained"] / 2.0 * 1e12)
    link = exchange_bytes_per_rank / (NVLINK_PEER_GBS * 1e9)
    target = max(compute, link)
    return {"bound": "tensor" if compute >= link else "nvlink", "compute_ms": compute * 1e3,
            "nvlink_ms": link * 1e3, "target_ms": target * 1e3, "measured_ms": seconds * 1e3,
            "frac": target / seconds,
            "peaks": f"TF32 {peaks['bf16_tflops_sustained'] / 2.0:.0f} TFLOP/s (measured bf16 / 2, "
                     f"sustained), NVLink {NVLINK_PEER_GBS:.0f} GB/s per direction (measured peer copy)"}


def cublas_tf32(torch, seconds: float = 4.0) -> dict:
    """cuBLAS TF32 (torch.matmul, allow_tf32) on 8192^3: best of 10 (burst) and back to
    back for `seconds` (sustained) -- the method of the driver's bf16 measurement, for the
    arithmetic these kernels actually use.  A yardstick beside the roofline denominator."""
    n = 8192
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        a = torch.rand(n, n, device="cuda") - 0.5
        b = torch.rand(n, n, device="cuda") - 0.5
        c = torch.empty(n, n, device="cuda")
        for _ in range(3):
            torch.matmul(a, b, out=c)
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch.matmul(a, b, out=c)
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1) * 1e-3)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        count = max(8, int(seconds / best))
        e0.record()
        for _ in range(count):
            torch.matmul(a, b, out=c)
        e1.record()
        torch.cuda.synchronize()
        sus = e0.elapsed_time(e1) * 1e-3 / count
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    flops = 2.0 * n ** 3
    return {"burst_tflops": flops / best / 1e12, "sustained_tflops": flops / sus / 1e12,
            "how": f"torch.matmul allow_tf32 {n}^3: best of 10, and {count} back to back"}


def sustained_segment(torch, info: dict, seconds: float, sampler: ClockSampler) -> dict:
    """At least `seconds` of back-to-back steps of an already warmed configuration, clocks
    sampled: what the kernel holds once the power limit has engaged."""
    per = info["seconds"]
    count = max(16, int(seconds / per))
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    info["many"](0, count)
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    return {"steps": count, "seconds": e0.elapsed_time(e1) * 1e-3, "clocks": clocks,
            "sec_per_step": e0.elapsed_time(e1) * 1e-3 / count}


def one_tile_gemm_us(torch, dev, k: int) -> float:
    """Microseconds per run, back to back, of a GEMM that is ONE 128 x 64 tile on one SM with a K
    of `k`, issued from C.  k = 32 (one K stage): what a launch of these kernels costs before
    any work (prologue, barriers, tensor memory allocation, one TMA round trip, epilogue).  A
    longer K adds only the time ONE SM needs to pull its operands into shared memory."""
    import xtc_b200.graphs.xtc.op as O
    from xtc_b200.backends.cuda import Backend
    from xtc_b200.backends.cuda.module import PlanHandle

    a = O.tensor((128, k), "float32", name="A")
    b = O.tensor((k, 64), "float32", name="B")
    with O.graph(name="floor") as gb:
        O.matmul(a, b, name="C")
    module = Backend(gb.graph).get_compiler(shared_lib=False).compile(None)
    # one CTA whatever k: name the tile and turn the library's K split off
    module.plan.steps[-1].config.update(tile_m=128, tile_n=64, tile_k=64, split_k=1)
    handle = PlanHandle(module.plan, dev)
    da, db, dc = (torch.zeros(128, k, device="cuda"), torch.zeros(k, 64, device="cuda"),
                  torch.zeros(128, 64, device="cuda"))
    ptrs = [da.data_ptr(), db.data_ptr(), dc.data_ptr()]
    stream = torch.cuda.current_stream().cuda_stream
    table = handle.pointer_sets([ptrs])
    total, _ = time_device_steps(torch, None, 400, 20,
                                 many=lambda first, count: handle.run_sets(table, first, count, stream))
    handle.close()
    return total / 400 * 1e6


def other_configs(torch, dev, args, peaks: dict, heavy: bool) -> dict:
    """Every other configuration, device-resident: the metric is per graph.  heavy = False:
    the short steps (measured before anything has run the chip into its power cap); heavy =
    True: c5 on one GPU, seconds of tensor work."""
    tf32_burst, _ = tf32_denominator(peaks, False)
    tf32_sus, _ = tf32_denominator(peaks, True)
    extra: dict = {}

    def tensor_entry(name, r, precision="tf32", sustained=False):
        c = r["cfg"]
        tf = c.flops / r["seconds"] / 1e12
        peak = (tf32_sus if sustained else tf32_burst) / (3.0 if precision == "3xtf32" else 1.0)
        return {"tflops": tf, "us": r["seconds"] * 1e6, "frac_of_tf32_peak": tf / peak,
                "peak": peak, "peak_kind": ("sustained" if sustained else "burst")
                + (" / 3 (three products per FMA)" if precision == "3xtf32" else "")}

    def guarded(key, fn):
        try:
            extra[key] = fn()
        except Exception as e:  # keep the headline line even if a side measurement fails
            extra[key] = {"error": f"{type(e).__name__}: {e}"}
        torch.cuda.empty_cache()

    def c1():
        r = bench_graph_device(torch, dev, "c1", max(args.steps, 400), args.warmup)
        out = tensor_entry("c1", r)
        c = r["cfg"]
        # c1 is 0.27 GFLOP over 3.7 MB: neither the tensor pipe (0.3 us) nor HBM (0.6 us)
        # bounds it.  What does: the cost of a launch of these kernels (a one-tile, one-stage
        # GEMM back to back) plus the time one SM needs to pull the operands of its piece
        # into shared memory, at the rate a one-tile GEMM with a long K shows
        floor = one_tile_gemm_us(torch, dev, 32)
        k_long = 1024
        fill_rate = (128 + 64) * (k_long - 32) * 4 / (one_tile_gemm_us(torch, dev, k_long) - floor)  # B/us
        m, k = c.input_shapes[0]
        n = c.input_shapes[1][1]
        kc = r["plan"].steps[-1].config  # the schedule the configuration ships
        pieces = max(1, kc.get("split_k", 1))
        rows = 128  # per CTA, also for a 256-row tile of a CTA pair
        cols = kc["tile_n"] // (2 if kc["tile_m"] == 256 else 1)
        cta_bytes = (rows + cols) * (k / pieces) * 4
        bound = floor + cta_bytes / fill_rate
        out["bound"] = {"kind": "launch + one SM's operand fill", "launch_floor_us": floor,
                        "sm_fill_gbs": fill_rate * 1e-3, "operand_bytes_per_cta": cta_bytes,
                        "tile": [kc["tile_m"], kc["tile_n"]], "k_pieces": pieces,
                        "bound_us": bound,
                        "tensor_us": c.flops / (tf32_burst * 1e12) * 1e6,
                        "hbm_us": c.bytes / (peaks["hbm_gbs"] * 1e9) * 1e6,
                        "frac_of_bound": bound / (r["seconds"] * 1e6)}
        return out

    if not heavy:
        guarded("c1", c1)
    if not heavy:
        guarded("c3", lambda: tensor_entry("c3", bench_graph_device(torch, dev, "c3", max(args.steps, 200), args.warmup)))
    if not heavy:
        guarded("c4", lambda: tensor_entry("c4", bench_graph_device(torch, dev, "c4", max(args.steps, 50), args.warmup)))

    def hbm_entry(name):
        r = bench_graph_device(torch, dev, name, max(args.steps, 100), args.warmup)
        gbs = r["cfg"].bytes / r["seconds"] / 1e9
        return {"gbs": gbs, "us": r["seconds"] * 1e6, "frac_of_hbm_peak": gbs / peaks["hbm_gbs"],
                "peak": peaks["hbm_gbs"], "bytes": r["cfg"].bytes}

    for name in (() if heavy else ("c4a", "relu512", "pad512")):
        guarded(name, lambda name=name: hbm_entry(name))

    # c5 on one GPU, device-resident: TF32 and 3xTF32 (seconds-long tensor work: sustained peak)
    def c5(precision):
        from xtc_b200 import configs

        a, b = configs.inputs("c5")
        dins = [torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()]
        del a, b
        steps = 20 if precision == "tf32" else 8
        r = bench_graph_device(torch, dev, "c5", steps, 3, precision=precision, device_inputs=dins)
        out = tensor_entry("c5", r, precision, sustained=True)
        out["steps"] = steps
        return out

    # a few layers of the reference's operation tables with nothing scheduled (the library's
    # own choice of kernel), through the evaluator's timing loop: one image / one token row
    def named_layers():
        from xtc_b200.backends.cuda import Backend
        from xtc_b200.search import Exploration, ExplorationConfig

        from xtc_b200 import artifacts

        out = {}
        layers = [(operator, name, None) for operator, name in (
            ("conv2d", "ResNet18_01"), ("conv2d", "Yolo9000_18"), ("matmul", "AlexNet_FC7"),
            ("matmul", "Gemma2B_QK"), ("matmul", "Llama3_In"))]
        # the reference's ResNet layers at the batch of c3 (its table holds one image each)
        for name in ("ResNet18_02", "ResNet18_06", "ResNet18_09"):
            dims = artifacts.operation_dims("conv2d", name)
            layers.append(("conv2d", f"{name}_batch32", [32] + dims[1:]))
        for operator, name, dims in layers:
            exp = Exploration(ExplorationConfig(operator=operator, op_name=None if dims else name, dims=dims,
                                                peak_flops=1e15))
            impl = Backend(exp.graph)
            module = impl.get_compiler(shared_lib=False).compile(impl.get_scheduler().schedule())
            times, code, msg = module.get_evaluator(repeat=3, number=50, min_repeat_ms=0).evaluate()
            if code != 0:
                out[name] = {"error": msg}
                continue
            sec = min(times)
            out[name] = {"us": sec * 1e6, "tflops": 2.0 * exp.fma_count() / sec / 1e12}
        return out

    if not heavy:
        guarded("named_layers_default_schedule", named_layers)
    else:
        guarded("c5_n1_tf32", lambda: c5("tf32"))
        guarded("c5_n1_3xtf32", lambda: c5("3xtf32"))
    return extra


def run_single(args) -> None:
    import torch

    from xtc_b200.runtimes.cuda import CudaDevice

    torch.cuda.set_device(0)
    dev = CudaDevice(0)
    dev.activate()
    workload = args.workload or "c2"
    peaks = measured_peaks()
    sampler = ClockSampler(0)

    # ---- device-resident throughput ("value") --------------------------------
    sampler.start()
    info = bench_graph_device(torch, dev, workload, args.steps, args.warmup,
                              precision=args.precision,
                              fuse_transpose=False if args.unfused_transpose else None)
    clocks = sampler.stop()
    cfg, plan = info["cfg"], info["plan"]
    sec = info["seconds"]
    launches_per_step = len(plan.steps) + (2 if args.precision == "3xtf32" else 0)

    # ---- end to end through host buffers ("e2e") ------------------------------
    e2e = None if args.no_e2e else measure_e2e(torch, dev, info["handle"], cfg, workload, args.steps)

    unit_work = cfg.flops if cfg.flops else cfg.bytes
    scale = 1e12 if cfg.flops else 1e9
    unit = "TFLOP/s" if cfg.flops else "GB/s"
    line = {
        "metric": "graph_throughput", "value": unit_work / sec / scale, "unit": unit,
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": ("f32" if not cfg.flops else "tf32" if args.precision == "tf32" else args.precision),
        "data": "synthetic",
        "config": {"workload": workload_name(workload), "precision": args.precision,
                   "kernel_config": plan.steps[-1].config, "fused": [list(s.fused) for s in plan.steps],
                   "l2": f"inputs rotate over {info['n_sets']} buffer sets of "
                         f"{info['set_bytes'] / 1e6:.0f} MB (> 126 MB L2 in total)"},
        "roofline": roofline_of(cfg, statistics.median(info["per_step"]), peaks, workload,
                                sustained=sec * args.steps > 1.0, precision=args.precision),
        "e2e": None if e2e is None else {
            "value": unit_work / e2e["sec"] / scale, "unit": unit, "h2d_bytes_per_step": e2e["h2d"],
            "d2h_bytes_per_step": e2e["d2h"], "ms_per_step": e2e["sec"] * 1e3, "steps": e2e["steps"],
            "api": "xtc_cuda_pipeline_submit/wait, depth 3 (pinned host buffers)",
            "synchronous_ms_per_step": e2e["sync_sec"] * 1e3,
            "synchronous_api": "xtc_cuda_plan_run_host"},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks,
    }
    # Order: everything short first, while the chip still clocks as it did for the headline;
    # then the runs that take it into the power cap (the cuBLAS yardstick, this kernel for a
    # second or more, c5 on one GPU), after which it stays at the capped clock for a while.
    extra = not args.no_extra and workload == "c2"
    if extra:
        line["other_configs"] = other_configs(torch, dev, args, peaks, heavy=False)
        try:
            yard = cublas_tf32(torch)
            line["tf32_cublas"] = yard
            line["roofline"]["frac_of_cublas_tf32_burst"] = line["roofline"]["achieved"] / yard["burst_tflops"]
        except Exception as e:
            line["tf32_cublas"] = {"error": str(e)}
    # ---- the same kernel for a second or more: sustained clocks ---------------
    if not args.no_extra and cfg.flops:
        seg = sustained_segment(torch, info, 1.2, ClockSampler(0))
        sus = roofline_of(cfg, seg["sec_per_step"], peaks, workload, sustained=True,
                          precision=args.precision)
        line["value_sustained"] = unit_work / seg["sec_per_step"] / scale
        line["sustained"] = {"steps": seg["steps"], "seconds": seg["seconds"],
                             "ms_per_step": seg["sec_per_step"] * 1e3, "clocks": seg["clocks"],
                             "roofline": sus}
        if "sustained_tflops" in line.get("tf32_cublas", {}):
            line["sustained"]["roofline"]["frac_of_cublas_tf32_sustained"] = (
                line["value_sustained"] / line["tf32_cublas"]["sustained_tflops"])
    del info
    torch.cuda.empty_cache()
    if extra:
        line["other_configs"].update(other_configs(torch, dev, args, peaks, heavy=True))
    # ---- CPU baseline ---------------------------------------------------------
    if not args.no_cpu:
        base = time_cpu(workload, 3, 1)
        base.pop("seconds_per_sample")
        line["cpu_baseline"] = base
    print(json.dumps(line), flush=True)


def run_sharded(args, rank: int, world: int, local_rank: int) -> None:
    import torch
    import torch.distributed as dist

    from xtc_b200 import configs
    from xtc_b200.backends.cuda.module import PlanHandle
    from xtc_b200.dist import BatchSharded, RowShardedMatmul
    from xtc_b200.runtimes.cuda import CudaDevice

    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    dev = CudaDevice(local_rank)
    dev.activate()
    workload = args.workload or "c5"
    peaks = measured_peaks()
    stream = torch.cuda.current_stream().cuda_stream
    sampler = ClockSampler(local_rank)
    checks: dict = {}
    nccl_rows = None

    def barrier() -> None:
        dist.barrier()

    if workload == "c5":
        M, K, N = 65536, 8192, 8192
        rows = M // world
        row_lo = rank * rows
        cfg = configs.build("c5", rows=rows)
        module = configs.compile_config(cfg, precision=args.precision)
        handle = PlanHandle(module.plan, dev)
        # the seeded inputs of the configuration: this rank's rows of A, all of B
        host_a, host_b = configs.input_rows("c5", row_lo, row_lo + rows)
        a_blk = torch.from_numpy(host_a).cuda()
        b = torch.from_numpy(host_b).cuda()
        c_full = torch.empty(M, N, device="cuda") if args.exchange == "nccl" else None
        c_blk = torch.empty(rows, N, device="cuda")  # target of the compute-only timing

        def compute(lo: int, hi: int, _stream) -> None:
            if hi - lo == rows:
                handle.run([a_blk.data_ptr(), b.data_ptr(), c_full[lo:hi].data_ptr()], stream)
            else:
                chunk_handles[(hi - lo)].run(
                    [a_blk[lo - row_lo: hi - row_lo].data_ptr(), b.data_ptr(), c_full[lo:hi].data_ptr()], stream)

        chunk_handles = {}
        if args.chunks > 1 and args.exchange == "nccl":
            from xtc_b200.dist import chunk_ranges
            for lo, hi in chunk_ranges(row_lo, row_lo + rows, args.chunks):
                if (hi - lo) not in chunk_handles:
                    ccfg = configs.build("c5", rows=hi - lo)
                    chunk_handles[hi - lo] = PlanHandle(
                        configs.compile_config(ccfg, precision=args.precision).plan, dev)
        peer_op = None
        if args.exchange != "nccl":
            from xtc_b200.dist import PeerStoreMatmul, PipelinedPeerMatmul
            gemm_cfg = dict(module.plan.steps[-1].config)
            if args.exchange in ("pipeline", "auto"):
                op = peer_op = PipelinedPeerMatmul(dev, a_blk.data_ptr(), b.data_ptr(), M, N, K, world, rank,
                                                   config=gemm_cfg)
                sharding = (f"rows of A and C split over {world} ranks, B replicated; each rank's rows go to "
                            "every peer's C by peer-to-peer copies (copy engines over NVLink) while the next "
                            "step's GEMM runs (exchange one step behind, two C buffers)"
                            if world > 1 else "one rank holds all rows (no exchange)")
            else:
                op = peer_op = PeerStoreMatmul(dev, a_blk.data_ptr(), b.data_ptr(), M, N, K, world, rank,
                                               config=gemm_cfg,
                                               exchange=args.exchange)
                how = ("one multicast store per vector through an NVLink multicast object (NVLS)"
                       if peer_op.exchange == "multimem" else "one 128-bit store per peer")
                sharding = (f"rows of A and C split over {world} ranks, B replicated; copier warps of the GEMM "
                            f"write each C tile into every rank's C over NVLink, {how} (fused all-gather)"
                            if world > 1 else "one rank holds all rows (no exchange)")
        else:
            from xtc_b200.dist import NcclRows
            nccl_rows = NcclRows(dev, world, rank) if world > 1 else None
            op = RowShardedMatmul(c_full, world, rank, compute, chunks=args.chunks, comm=nccl_rows)
            sharding = (f"rows of A and C split over {world} ranks, B replicated, NCCL all-gather of C "
                        "(xtc_cuda_allgather_rows)")
        step = lambda i: op.step(stream)
        total_flops = 2 * M * N * K
        local_cfg = cfg
        h2d = a_blk.numel() * 4
        d2h = rows * N * 4
        launches = 1 if (args.chunks <= 1 or args.exchange != "nccl") else args.chunks
        if world > 1 and args.exchange in ("pipeline", "auto"):
            launches = 2  # the GEMM and the one-warp barrier; the copies are the copy engines'
        exchange_bytes = rows * N * 4 * (world - 1)  # the rank's block of C, to every other rank
    elif workload == "c3":
        sh = BatchSharded(32, world, rank)
        cfg = configs.build("c3", batch=sh.local_batch)
        module = configs.compile_config(cfg)
        handle = PlanHandle(module.plan, dev)
        x_all, w_np = configs.inputs("c3")
        x = torch.from_numpy(x_all[sh.lo:sh.hi]).cuda()
        w = torch.from_numpy(w_np).cuda()
        # enough buffer sets that a step never finds its input in L2, whatever the shard's size
        n_sets = int(min(max(8, math.ceil(3 * L2_BYTES / (2 * x.numel() * 4))), 64))
        xs = [x.clone() for _ in range(n_sets)]
        ys = [torch.empty(cfg.output_shape, device="cuda") for _ in range(n_sets)]
        ptr_sets = [[xs[i].data_ptr(), w.data_ptr(), ys[i].data_ptr()] for i in range(n_sets)]
        table = handle.pointer_sets(ptr_sets)
        step = lambda i: handle.run(ptr_sets[i % n_sets], stream)
        # a shard's step is a few microseconds: issue the steps from C, not one call each
        step_many = lambda first, count: handle.run_sets(table, first, count, stream)
        step_many(0, n_sets)  # every set visited once before the warm-up proper
        total_flops = configs.build("c3").flops
        local_cfg = cfg
        h2d = x.numel() * 4 + w.numel() * 4
        d2h = ys[0].numel() * 4
        launches = 1
        exchange_bytes = 0
        sharding = f"batch of 32 split over {world} ranks, no collective"
    else:
        raise SystemExit(f"workload {workload} does not shard; run it with plain `python bench.py`")

    if rank == 0:
        sampler.start()
    total, per = time_device_steps(torch, step, args.steps, args.warmup, barrier,
                                   many=step_many if workload == "c3" else None)
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([total], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    sec = float(t.item()) / args.steps
    status = dev.status()

    # ---- outside the timed region: is the gathered C right? ---------------------------
    if workload == "c5":
        # this rank recomputes, in float64 on the host, a few rows that ANOTHER rank produced
        # (from the seeded inputs of that rank's block) and compares them with its own copy
        peer = (rank + 1) % world
        pick = np.sort(np.random.default_rng(100 + rank).choice(rows, 4, replace=False))
        peer_rows = peer * rows + pick
        a_peer = np.stack([configs.input_rows("c5", int(r), int(r) + 1)[0][0] for r in peer_rows])
        want = a_peer.astype(np.float64) @ host_b.astype(np.float64)
        torch.cuda.synchronize()
        if peer_op is not None:
            got = np.empty((4, N), np.float32)
            for i, r in enumerate(peer_rows):
                dev.memory_copy_from(_ptr(peer_op.c_local.value + int(r) * N * 4), got[i], N * 4)
        else:
            got = c_full[torch.from_numpy(peer_rows).cuda()].cpu().numpy()
        err = float(np.abs(got - want).max() / np.abs(want).max())
        checks = {"gathered_rows_checked": [int(r) for r in peer_rows], "from_rank": peer,
                  "rel_err_vs_float64": err, "tolerance": 1e-2 if args.precision == "tf32" else 1e-5}
        ok = torch.tensor([1.0 if err <= checks["tolerance"] else 0.0], device="cuda")
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        checks["all_ranks_ok"] = bool(ok.item() == 1.0)
        assert checks["all_ranks_ok"], f"gathered rows differ from the recomputation: {checks}"

    # compute-only time of the local block (no exchange), for the roofline line
    if workload == "c5":
        comp_total, comp_per = time_device_steps(
            torch, lambda i: handle.run([a_blk.data_ptr(), b.data_ptr(), c_blk.data_ptr()], stream),
            max(3, min(args.steps, 10)), 1, barrier)
    else:
        comp_total, comp_per = time_device_steps(torch, step, max(3, args.steps), 1, barrier,
                                                 many=step_many)
    kernel_sec = statistics.median(comp_per)
    t = torch.tensor([kernel_sec], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    kernel_sec_max = float(t.item())

    # end to end: the rank's inputs from pinned host memory, its result block back
    e2e_steps = 4
    if workload == "c5" and peer_op is not None:
        pin_a = torch.from_numpy(host_a).pin_memory()
        pin_c = torch.empty(rows, N).pin_memory()
        loop = peer_op.host_loop()
        e2e_api = (f"{type(peer_op).__name__}.host_loop(): submit / wait (xtc_cuda_memcpy_*, events, "
                   + ("xtc_cuda_gemm_f32 + peer copies + xtc_cuda_peer_barrier)"
                      if args.exchange in ("pipeline", "auto") else "xtc_cuda_gemm_f32_bcast)"))

        def e2e_run(n: int) -> None:
            for _ in range(n):
                loop.submit(pin_a.data_ptr(), pin_c.data_ptr())
            loop.wait()
    elif workload == "c5":
        pin_a = torch.from_numpy(host_a).pin_memory()
        pin_c = torch.empty(rows, N).pin_memory()
        e2e_api = "copies + RowShardedMatmul.step (NCCL all-gather), synchronous"

        def e2e_run(n: int) -> None:
            for _ in range(n):
                a_blk.copy_(pin_a, non_blocking=True)
                op.step(stream)
                pin_c.copy_(c_full[row_lo:row_lo + rows], non_blocking=True)
                torch.cuda.synchronize()
    else:
        host_x = pinned_like(dev, x_all[sh.lo:sh.hi])
        host_w = pinned_like(dev, w_np)
        host_ys = [pinned_like(dev, np.zeros(cfg.output_shape, np.float32)) for _ in range(3)]
        pipe = handle.pipeline(depth=3)
        e2e_steps = 30
        e2e_api = "xtc_cuda_pipeline_submit/wait, depth 3 (pinned host buffers)"

        def e2e_run(n: int) -> None:
            for i in range(n):
                pipe.submit([host_x, host_w, host_ys[i % 3]])
            pipe.wait()
    e2e_run(2)
    barrier()
    t0 = time.perf_counter()
    e2e_run(e2e_steps)
    barrier()
    e2e_local = (time.perf_counter() - t0) / e2e_steps
    t = torch.tensor([e2e_local], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_sec = float(t.item())
    if workload == "c5" and peer_op is not None:
        checks["e2e_block_equals_device_block"] = bool(
            np.array_equal(pin_c[:4].numpy(), _rows_of(dev, peer_op.c_block, 4, N)))

    # the same workload on ONE GPU (rank 0 alone), so that the line carries both ends of the curve
    single = None
    if workload == "c5" and world > 1 and rank == 0 and not args.no_extra:
        try:
            if peer_op is not None:
                pass  # its C stays mapped by the peers until close(); memory is plentiful
            full_a, _ = configs.inputs("c5")
            dins = [torch.from_numpy(full_a).cuda(), b]
            del full_a
            r = bench_graph_device(torch, dev, "c5", 10, 3, precision=args.precision, device_inputs=dins)
            single = {"ms_per_step": r["seconds"] * 1e3, "value": total_flops / r["seconds"] / 1e12,
                      "unit": "TFLOP/s", "steps": 10,
                      "what": "the whole 65536-row product on rank 0's GPU alone, device-resident"}
            del r, dins
        except Exception as e:
            single = {"error": f"{type(e).__name__}: {e}"}
    barrier()

    if rank == 0:
        line = {
            "metric": "graph_throughput", "value": total_flops / sec / 1e12, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "tf32" if args.precision == "tf32" else args.precision, "data": "synthetic",
            "config": {"workload": workload_name(workload), "sharding": sharding,
                       "chunks": args.chunks,
                       "exchange": ((peer_op.exchange if peer_op is not None else "nccl") if world > 1
                                    else "none") if workload == "c5" else "none",
                       "kernel_config": module.plan.steps[-1].config,
                       "inputs": "the configuration's seeded inputs (each rank draws its own rows)",
                       "l2": "per-rank operands (>= 0.5 GB) exceed the 126 MB L2"
                             if workload == "c5" else
                             f"inputs rotate over {n_sets} buffer sets (> 126 MB L2 in total)"},
            "roofline": roofline_of(local_cfg, kernel_sec, peaks, workload, sustained=True,
                                    precision=args.precision),
            "compute_only_ms": kernel_sec * 1e3,
            "compute_only": {"ms_per_step_max_over_ranks": kernel_sec_max * 1e3,
                             "value": total_flops / kernel_sec_max / 1e12, "unit": "TFLOP/s",
                             "what": "every rank's block product without the exchange"},
            "fused_roofline": fused_roofline(total_flops / world, exchange_bytes, sec, peaks),
            "e2e": {"value": total_flops / e2e_sec / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                    "ms_per_step": e2e_sec * 1e3, "steps": e2e_steps, "api": e2e_api,
                    "note": "per rank: own input block in, own result block out; the input copy of the "
                            "next step overlaps the output copy of this one"},
            "checks": checks,
            "gpu_launches": launches * args.steps,
            "clocks": clocks, "device_status": status,
        }
        if single is not None:
            line["single_gpu_same_workload"] = single
        if not args.no_cpu and world == 1:
            base = time_cpu(workload, 3, 1)
            base.pop("seconds_per_sample")
            line["cpu_baseline"] = base
        print(json.dumps(line), flush=True)
    dist.barrier()
    if workload == "c5" and peer_op is not None:
        loop.close()
        peer_op.close()
    if nccl_rows is not None:
        dist.barrier()
        nccl_rows.close()
    dist.destroy_process_group()


def _ptr(address: int):
    import ctypes

    return ctypes.c_void_p(address)


def _rows_of(dev, address: int, n_rows: int, n: int) -> np.ndarray:
    out = np.empty((n_rows, n), np.float32)
    dev.memory_copy_from(_ptr(address), out, out.nbytes)
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None,
                    choices=["c1", "c2", "c3", "c4", "c4a", "c5", "relu512", "pad512"])
    ap.add_argument("--precision", default="tf32", choices=["tf32", "3xtf32", "fp32"])
    ap.add_argument("--unfused-transpose", action="store_true",
                    help="c4: run the transpose as its own kernel instead of reading A transposed")
    ap.add_argument("--chunks", type=int, default=1, help="row chunks overlapped with the exchange (N>1)")
    ap.add_argument("--exchange", default="auto", choices=["auto", "multimem", "peer", "pipeline", "nccl"],
                    help="c5 at N>1: the exchange one step behind the product, by peer-to-peer copies on "
                         "the copy engines (pipeline; what auto picks: the fastest as measured on 2 and "
                         "8 GPUs), the all-gather fused into the GEMM by one store per peer (peer) or by "
                         "NVLink multicast stores (multimem), or GEMM followed by an NCCL all-gather (nccl)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-extra", action="store_true", help="skip the other configurations")
    ap.add_argument("--no-e2e", action="store_true",
                    help="skip the host-buffer leg (for profiler runs; the line then has e2e null)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    # built library is required: fail loudly, never fall back
    from xtc_b200 import capi
    capi.load()
    if world == 1 and not under_torchrun():
        if args.gpus != 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
        run_single(args)
    else:
        run_sharded(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
