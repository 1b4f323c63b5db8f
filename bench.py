#!/usr/bin/env python
"""Benchmark of the CUDA backend on the five benchmark graphs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1..c5] [--impl reference]

N == 1 (default workload c2, matmul 4096^3 + relu): one step = one run of the
compiled graph.  N > 1 (launched by torchrun, default workload c5, the
row-sharded 65536x8192x8192 matmul): one step = every rank computes its row
block and the blocks are all-gathered; total work is fixed ("strong" scaling).
Prints ONE JSON line on rank 0.

  value     graph throughput with inputs resident in device memory
  e2e       the same through host buffers: pinned host -> device copies of the
            inputs and a device -> host copy of the result inside the timed region
  roofline  the dominant kernel's achieved rate against the measured peak
  cpu_baseline / --impl reference
            the CPU loop-nest restatement of the reference's MLIR llvmir lowering
            (oracle/cpu_loopnest.c) on the host cores
"""

from __future__ import annotations

import argparse
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
NCU_TRAFFIC = {"c1": None, "c2": 395.1e6, "c3": 25.9e6, "c4": None, "c4a": 488.1e6, "c5": None}


def measured_peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "source": "MEASURED_PEAKS.json (of measured)"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "recipe fallback (of fallback)"}


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
    """(inputs, description, fraction of the full workload) of the bounded CPU sample."""
    from xtc_b200 import configs

    if workload == "c5":
        rows = 1024  # 1/64 of the rows; time scales linearly with rows
        rng = np.random.default_rng(4)
        a = rng.uniform(-1, 1, (rows, 8192)).astype(np.float32)
        b = rng.normal(0, 1 / np.sqrt(8192), (8192, 8192)).astype(np.float32)
        return [a, b], f"rows 0..{rows} of A (1/64 of the work), all of B", rows / 65536
    if workload == "c4":
        return configs.inputs("c4"), "the full graph (transpose + matmul)", 1.0
    return configs.inputs(workload), "the full workload", 1.0


def time_cpu(workload: str, steps: int, warmup: int) -> dict:
    """Times the CPU loop nests on all host cores; TFLOP/s of the full workload."""
    from oracle import cpu_baseline as cb
    from xtc_b200 import configs

    cfg = configs.build(workload)
    ins, desc, frac = cpu_sample(workload)
    for _ in range(max(warmup, 1)):
        cb.run_config(workload, ins)
    times = []
    for _ in range(max(steps, 1)):
        t0 = time.perf_counter()
        cb.run_config(workload, ins)
        times.append(time.perf_counter() - t0)
    t = min(times)
    work, unit = (cfg.flops / 1e12, "TFLOP/s") if cfg.flops else (cfg.bytes / 1e9, "GB/s")
    return {"value": work * frac / t, "unit": unit, "cores": cb.threads(),
            "kind": "port", "sample": f"{desc}; best of {len(times)} runs, {t * 1e3:.1f} ms each",
            "seconds_per_sample": t}


def run_reference(args, rank: int, world: int) -> None:
    if rank != 0:
        return
    workload = args.workload or ("c2" if world == 1 else "c5")
    steps = min(args.steps, 5)
    warm = min(args.warmup, 1)
    base = time_cpu(workload, steps, warm)
    t = base.pop("seconds_per_sample")
    line = {
        "impl": "reference", "metric": "graph_throughput", "value": base["value"],
        "unit": base["unit"], "n_gpus": world, "steps": steps, "warmup": warm,
        "ms_per_step": t * 1e3, "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": workload_name(workload)},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": base["unit"], "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "note": ("the reference's MLIR llvmir backend cannot be built on this box (no MLIR/LLVM "
                 "toolchain); this is its loop nest restated in C, OpenMP over the host cores"),
    }
    print(json.dumps(line), flush=True)


def workload_name(w: str) -> str:
    return {
        "c1": "c1: matmul 512x1024x256 f32",
        "c2": "c2: matmul 4096^3 + relu f32 (configs[1])",
        "c3": "c3: pad + conv2d 3x3 + relu, NHWC 32x56x56x64 -> 64 f32",
        "c4": "c4: transpose 8192^2 + matmul 8192x8192x1024 f32",
        "c4a": "c4a: transpose 8192^2 f32 alone",
        "c5": "c5: row-sharded matmul 65536x8192x8192 f32 + all-gather",
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


def time_device_steps(torch, fn, steps: int, warmup: int, barrier=None):
    """W warm-up calls, then K calls bracketed by synchronize (+ barrier); returns
    (total seconds, list of average seconds per call of each timed segment), both
    from events on the current stream."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    if barrier:
        barrier()
    # An event between two launches costs a few microseconds of stream time, which is
    # not negligible next to a 10-30 us step: record one every `stride` steps (at most
    # 16 segments) and report each segment's average step time.
    stride = max(1, -(-steps // 16))
    marks = list(range(0, steps, stride)) + [steps]
    evs = [torch.cuda.Event(enable_timing=True) for _ in marks]
    torch.cuda.synchronize()
    evs[0].record()
    nxt = 1
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
                       fuse_transpose=None, device_inputs=None):
    """Device-resident throughput of one configuration on the current GPU."""
    from xtc_b200 import configs
    from xtc_b200.backends.cuda.module import PlanHandle

    cfg = configs.build(name)
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
    sets = []
    for s in range(n_sets):
        ins = device_inputs if s == 0 else [t.clone() for t in device_inputs]
        out = torch.empty(cfg.output_shape, dtype=torch.float32, device="cuda")
        sets.append(([t.data_ptr() for t in ins] + [out.data_ptr()], ins, out))
    stream = torch.cuda.current_stream().cuda_stream

    def step(i: int) -> None:
        handle.run(sets[i % n_sets][0], stream)

    # every buffer set is visited once before timing (first visits record the CUDA graph)
    total, per = time_device_steps(torch, step, steps, max(warmup, n_sets))
    assert dev.status() == 0, "a kernel reported a bounded-wait timeout"
    info = {"cfg": cfg, "plan": plan, "seconds": total / steps, "per_step": per,
            "n_sets": n_sets, "set_bytes": set_bytes, "handle": handle, "sets": sets}
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


def roofline_of(cfg, seconds: float, peaks: dict, workload: str, sustained: bool) -> dict:
    if cfg.bound == "hbm":
        achieved = cfg.bytes / seconds / 1e9
        return {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "traffic": NCU_TRAFFIC.get(workload),
                "peak_source": peaks["source"]}
    bf16 = peaks["bf16_tflops_sustained"] if sustained else peaks["bf16_tflops"]
    peak = bf16 / 2.0  # kind::tf32 issues at half the bf16 rate
    achieved = cfg.flops / seconds / 1e12
    return {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
            "frac": achieved / peak, "traffic": NCU_TRAFFIC.get(workload),
            "peak_source": peaks["source"] + ": dense bf16 / 2 for TF32 ("
                           + ("sustained" if sustained else "burst") + ")"}


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


def run_single(args) -> None:
    import torch

    from xtc_b200 import configs
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
                                sustained=sec * args.steps > 1.0),
        "e2e": None if e2e is None else {
            "value": unit_work / e2e["sec"] / scale, "unit": unit, "h2d_bytes_per_step": e2e["h2d"],
            "d2h_bytes_per_step": e2e["d2h"], "ms_per_step": e2e["sec"] * 1e3, "steps": e2e["steps"],
            "api": "xtc_cuda_pipeline_submit/wait, depth 3 (pinned host buffers)",
            "synchronous_ms_per_step": e2e["sync_sec"] * 1e3,
            "synchronous_api": "xtc_cuda_plan_run_host"},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks,
    }
    # ---- the other configurations, device-resident, for context --------------
    if not args.no_extra and workload == "c2":
        extra = {}
        for name in ("c1", "c3", "c4"):
            try:
                r = bench_graph_device(torch, dev, name, max(args.steps, 200), args.warmup)
                c = r["cfg"]
                extra[name] = {"tflops": c.flops / r["seconds"] / 1e12, "us": r["seconds"] * 1e6,
                               "frac_of_tf32_peak": c.flops / r["seconds"] / 1e12 / (peaks["bf16_tflops"] / 2)}
                del r
            except Exception as e:  # keep the headline line even if a side measurement fails
                extra[name] = {"error": str(e)}
        line["other_configs"] = extra
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

    def barrier() -> None:
        dist.barrier()

    if workload == "c5":
        M, K, N = 65536, 8192, 8192
        rows = M // world
        cfg = configs.build("c5", rows=rows)
        module = configs.compile_config(cfg, precision=args.precision)
        handle = PlanHandle(module.plan, dev)
        gen = torch.Generator(device="cuda").manual_seed(4 + rank)
        a_blk = torch.rand(rows, K, device="cuda", generator=gen) * 2 - 1
        genb = torch.Generator(device="cuda").manual_seed(4)
        b = torch.randn(K, N, device="cuda", generator=genb) / math.sqrt(8192)
        c_full = torch.empty(M, N, device="cuda") if args.exchange == "nccl" else None
        c_blk = torch.empty(rows, N, device="cuda")  # target of the compute-only timing
        row_lo = rank * rows

        def compute(lo: int, hi: int, _stream) -> None:
            if hi - lo == rows:
                handle.run([a_blk.data_ptr(), b.data_ptr(), c_full[lo:hi].data_ptr()], stream)
            else:
                chunk_handles[(hi - lo)].run(
                    [a_blk[lo - row_lo: hi - row_lo].data_ptr(), b.data_ptr(), c_full[lo:hi].data_ptr()], stream)

        chunk_handles = {}
        if args.chunks > 1:
            from xtc_b200.dist import chunk_ranges
            for lo, hi in chunk_ranges(row_lo, row_lo + rows, args.chunks):
                if (hi - lo) not in chunk_handles:
                    ccfg = configs.build("c5", rows=hi - lo)
                    chunk_handles[hi - lo] = PlanHandle(
                        configs.compile_config(ccfg, precision=args.precision).plan, dev)
        if args.exchange == "peer":
            from xtc_b200.dist import PeerStoreMatmul
            gemm_cfg = dict(module.plan.steps[-1].config)
            op = PeerStoreMatmul(dev, a_blk.data_ptr(), b.data_ptr(), M, N, K, world, rank,
                                 config=gemm_cfg)
            result_block_ptr = op.c_block
            sharding = (f"rows of A and C split over {world} ranks, B replicated; the GEMM epilogue "
                        f"stores each C tile into every rank's C over NVLink (fused all-gather)")
        else:
            op = RowShardedMatmul(c_full, world, rank, compute, chunks=args.chunks)
            result_block_ptr = c_full[row_lo:row_lo + rows].data_ptr()
            sharding = f"rows of A and C split over {world} ranks, B replicated, NCCL all-gather of C"
        step = lambda i: op.step(stream)
        total_flops = 2 * M * N * K
        local_cfg = cfg
        h2d = a_blk.numel() * 4
        d2h = rows * N * 4
        launches = 1 if (args.chunks <= 1 or args.exchange == "peer") else args.chunks
        exchange_bytes = rows * N * 4 * (world - 1)  # the rank's block of C, to every other rank
    elif workload == "c3":
        sh = BatchSharded(32, world, rank)
        cfg = configs.build("c3", batch=sh.local_batch)
        module = configs.compile_config(cfg)
        handle = PlanHandle(module.plan, dev)
        x_all, w_np = configs.inputs("c3")
        x = torch.from_numpy(x_all[sh.lo:sh.hi]).cuda()
        w = torch.from_numpy(w_np).cuda()
        n_sets = 8
        xs = [x.clone() for _ in range(n_sets)]
        ys = [torch.empty(cfg.output_shape, device="cuda") for _ in range(n_sets)]
        step = lambda i: handle.run([xs[i % n_sets].data_ptr(), w.data_ptr(), ys[i % n_sets].data_ptr()], stream)
        total_flops = configs.build("c3").flops
        local_cfg = cfg
        h2d = x.numel() * 4 + w.numel() * 4
        d2h = ys[0].numel() * 4
        launches = 1
        exchange_bytes = 0
        sharding = f"batch of 32 split over {world} ranks, no collective"
    else:
        raise SystemExit(f"workload {workload} does not shard; run it with --gpus 1")

    if rank == 0:
        sampler.start()
    total, per = time_device_steps(torch, step, args.steps, args.warmup, barrier)
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([total], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    sec = float(t.item()) / args.steps
    status = dev.status()

    # compute-only time of the local block (no exchange), for the roofline line
    comp_total, comp_per = time_device_steps(
        torch, lambda i: handle.run(
            [a_blk.data_ptr(), b.data_ptr(), c_blk.data_ptr()], stream)
        if workload == "c5" else step(i), max(3, min(args.steps, 10)), 1, barrier)
    kernel_sec = statistics.median(comp_per)

    # end to end: the rank's inputs from pinned host memory, its result block back
    e2e_steps = 4
    if workload == "c5":
        host_a = torch.empty(rows, K, pin_memory=True)
        host_c = torch.empty(rows, N, pin_memory=True)

        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        main = torch.cuda.current_stream()

        def e2e_run(n: int) -> None:
            """n steps; every step copies the rank's A block in and its C block out.  The
            input copy of step i+1 and the output copy of step i both follow the kernel of
            step i and run side by side (the link is full duplex)."""
            ev_in, ev_out, ev_run = torch.cuda.Event(), torch.cuda.Event(), torch.cuda.Event()
            with torch.cuda.stream(s_in):
                a_blk.copy_(host_a, non_blocking=True)
                ev_in.record(s_in)
            for i in range(n):
                main.wait_event(ev_in)       # this step's input has landed
                if i > 0:
                    main.wait_event(ev_out)  # the previous result is out before C is rewritten
                op.step(stream)
                ev_run.record(main)
                s_out.wait_event(ev_run)
                dev.lib.xtc_cuda_memcpy_d2h(host_c.data_ptr(), result_block_ptr, rows * N * 4,
                                            s_out.cuda_stream)
                ev_out.record(s_out)
                if i + 1 < n:
                    s_in.wait_event(ev_run)
                    with torch.cuda.stream(s_in):
                        a_blk.copy_(host_a, non_blocking=True)
                        ev_in.record(s_in)
            torch.cuda.synchronize()
    else:
        host_x = torch.empty(x.shape, pin_memory=True)
        host_y = torch.empty(cfg.output_shape, pin_memory=True)

        def e2e_run(n: int) -> None:
            for _ in range(n):
                xs[0].copy_(host_x, non_blocking=True)
                step(0)
                host_y.copy_(ys[0], non_blocking=True)
                torch.cuda.synchronize()
    e2e_run(1)
    barrier()
    t0 = time.perf_counter()
    e2e_run(e2e_steps)
    barrier()
    e2e_local = (time.perf_counter() - t0) / e2e_steps
    t = torch.tensor([e2e_local], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_sec = float(t.item())

    if rank == 0:
        line = {
            "metric": "graph_throughput", "value": total_flops / sec / 1e12, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "tf32" if args.precision == "tf32" else args.precision, "data": "synthetic",
            "config": {"workload": workload_name(workload), "sharding": sharding,
                       "chunks": args.chunks,
                       "exchange": args.exchange if workload == "c5" else "none", "kernel_config": module.plan.steps[-1].config,
                       "l2": "per-rank operands (>= 0.5 GB) exceed the 126 MB L2"
                             if workload == "c5" else "inputs rotate over 8 buffer sets"},
            "roofline": roofline_of(local_cfg, kernel_sec, peaks, workload, sustained=True),
            "compute_only_ms": kernel_sec * 1e3,
            "fused_roofline": fused_roofline(total_flops / world, exchange_bytes, sec, peaks),
            "e2e": {"value": total_flops / e2e_sec / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                    "ms_per_step": e2e_sec * 1e3, "steps": e2e_steps,
                    "note": "per rank: own input block in, own result block out; the input copy of the "
                            "next step overlaps the output copy of this one"},
            "gpu_launches": launches * args.steps,
            "clocks": clocks, "device_status": status,
        }
        print(json.dumps(line), flush=True)
    dist.barrier()
    dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=["c1", "c2", "c3", "c4", "c4a", "c5"])
    ap.add_argument("--precision", default="tf32", choices=["tf32", "3xtf32", "fp32"])
    ap.add_argument("--unfused-transpose", action="store_true",
                    help="c4: run the transpose as its own kernel instead of reading A transposed")
    ap.add_argument("--chunks", type=int, default=1, help="row chunks overlapped with the exchange (N>1)")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="c5 at N>1: fused peer stores in the GEMM epilogue, or an NCCL all-gather")
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
    if world == 1:
        if args.gpus != 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
        run_single(args)
    else:
        run_sharded(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
