#!/usr/bin/env python
"""Bench of the EXL3 projection hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (BASELINE.json configs[1], the decode-row half): the dense trunk sweep, shapes 2048x2048, 2048x6144 and
6144x2048 at K in {1,2,3,4,5,6,8} bits, one f16 activation row each: 21 linears a step, 106.4 MB of trellis code bytes.
Metric: code-byte GB/s = trellis bytes read per step / step time (the reference's byte convention: code bytes only).
Weights rotate over several copies larger than L2 together, so every step streams its codes from HBM.

Prints ONE JSON line (rank 0). `--impl reference` times the CPU restatement of the reference's host implementation
(format.project) on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SHAPES = [(2048, 2048), (2048, 6144), (6144, 2048)]
KS = [1, 2, 3, 4, 5, 6, 8]
METRIC = "decode_row_code_byte_throughput"
UNIT = "GB/s"
WORKLOAD = "configs[1] dense trunk sweep, decode rows: 3 shapes x K{1,2,3,4,5,6,8}, 1 f16 row, MUL1, +-1 signs"


def code_bytes(in_dim: int, out_dim: int, k: int) -> int:
    return in_dim * out_dim * k // 8


STEP_BYTES = sum(code_bytes(i, o, k) for (i, o) in SHAPES for k in KS)


def measured_peaks() -> tuple[float, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def host_operands(copy: int):
    """The sweep's 21 linears for weight copy `copy` as numpy arrays (seeded; BASELINE: seeded uniform codes, +-1 signs)."""
    from turboexl3_b200 import synth
    ops = []
    for si, (i, o) in enumerate(SHAPES):
        for k in KS:
            ops.append((i, o, 16 * k, *synth.linear(1000 * copy + 10 * si + k, i, o, 16 * k)))
    return ops


def cpu_sample(threads: int, reps: int = 1) -> dict:
    """The oracle's faithful format.project (every tile decoded per call) over one pass of the sweep, all host threads."""
    from oracle import binding as ob
    from turboexl3_b200 import synth
    ops = host_operands(0)
    xs = {i: synth.activations(7, 1, i).astype(np.float32) for i in (2048, 6144)}
    t0 = time.perf_counter()
    for _ in range(reps):
        for (i, o, n, trellis, suh, svh) in ops:
            ob.linear_rows(xs[i], trellis, suh, svh, i, o, n, ob.MUL1, 16, threads=threads)
    dt = (time.perf_counter() - t0) / reps
    return {"seconds_per_pass": dt, "value": STEP_BYTES / dt / 1e9}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import binding as ob
    ob.build()
    threads = ob.host_threads()
    for _ in range(max(0, min(args.warmup, 1))):
        cpu_sample(threads)
    times = []
    for _ in range(max(1, min(args.steps, 3))):
        times.append(cpu_sample(threads)["seconds_per_pass"])
    dt = statistics.mean(times)
    value = STEP_BYTES / dt / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": len(times), "warmup": min(args.warmup, 1), "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "note": "CPU restatement of the reference's format.project (oracle port); "
                   "the reference itself is Zig and cannot be built here"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": "one full pass of the 21-linear sweep per step, every tile decoded per call"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    import turboexl3_b200 as t3

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    t3.lib()

    copies = 3  # 3 x 106 MB of codes > the 126 MB L2
    sets = []
    for c in range(copies):
        dev_ops = []
        for (i, o, n, trellis, suh, svh) in host_operands(c):
            dev_ops.append((i, o, n, torch.from_numpy(trellis).cuda(), torch.from_numpy(suh).cuda(),
                            torch.from_numpy(svh).cuda()))
        sets.append(dev_ops)
    from turboexl3_b200 import synth
    x_host = {i: torch.from_numpy(synth.activations(7, 1, i)).pin_memory() for i in (2048, 6144)}
    x_dev = {i: v.cuda() for i, v in x_host.items()}
    y_host = {o: torch.empty((1, o), dtype=torch.float16).pin_memory() for o in (2048, 6144)}
    dec = t3.Decode.mul1

    def step_eager(s: int):
        for (i, o, n, t, a, b) in sets[s % copies]:
            t3.linear(x_dev[i], t, a, b, dec)

    # One CUDA graph per weight copy: the 21 launches of a step replay without host work between them. The launches
    # carry the programmatic-dependent-launch attribute, so a linear's weight streaming overlaps its predecessor's tail.
    graphs = []
    launch_mode = "cuda graph per step (21 kernel nodes)"
    if not args.eager:
        try:
            for c in range(copies):
                step_eager(c)
            torch.cuda.synchronize()
            for c in range(copies):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    step_eager(c)
                graphs.append(g)
        except Exception as exc:  # capture refused: time the eager launches and say so
            graphs = []
            launch_mode = f"eager launches (graph capture failed: {type(exc).__name__})"
            torch.cuda.synchronize()
    else:
        launch_mode = "eager launches"
    per_step_launches = len(sets[0])

    def step_device(s: int):
        if graphs:
            graphs[s % copies].replay()
        else:
            step_eager(s)

    def step_e2e(s: int):
        last = None
        for (i, o, n, t, a, b) in sets[s % copies]:
            xd = x_host[i].cuda(non_blocking=True)
            y = t3.linear(xd, t, a, b, dec)
            y_host[o].copy_(y, non_blocking=True)
            last = y
        torch.cuda.current_stream().synchronize()
        return last

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    warm = max(args.warmup, 3)
    for s in range(warm):
        step_device(s)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = t3.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for s in range(args.steps):
        step_device(warm + s)
    ev1.record()
    barrier()
    ms = ev0.elapsed_time(ev1)
    launches = (t3.launch_count() - launches0) if not graphs else per_step_launches * args.steps

    # end to end: host buffers in, host buffers out, copies inside the timed region
    for s in range(2):
        step_e2e(s)
    barrier()
    t0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for s in range(args.steps):
        step_e2e(warm + s)
    e1.record()
    barrier()
    e2e_ms = max(e0.elapsed_time(e1), 0.0)
    e2e_wall_ms = (time.perf_counter() - t0) * 1e3
    clocks = sampler.stop() if rank == 0 else None

    # per-case kernel times (events around repeats of one linear on rotating copies)
    cases = {}
    if rank == 0 and not args.no_cases:
        for idx, (i, o, n, _, _, _) in enumerate(sets[0]):
            reps = 10
            def burst():
                for r in range(copies):
                    t3.linear(x_dev[i], *sets[r][idx][3:], dec)
            burst()
            torch.cuda.synchronize()
            cg = None
            if graphs:
                cg = torch.cuda.CUDAGraph()
                with torch.cuda.graph(cg):
                    burst()
            run = cg.replay if cg is not None else burst
            run()
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a0.record()
            for r in range(reps):
                run()
            a1.record()
            torch.cuda.synchronize()
            us = a0.elapsed_time(a1) * 1e3 / (reps * copies)
            cases[f"{i}x{o}_K{n // 16}"] = {"us": round(us, 2), "GBps": round(code_bytes(i, o, n // 16) / us / 1e3, 1)}

    if t3.device_error() != 0:
        raise SystemExit("a kernel reported a bounded-wait failure; the numbers are void")

    times = torch.tensor([ms, e2e_ms, e2e_wall_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms, e2e_wall_ms = times.tolist()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_peaks()
    ms_per_step = ms / args.steps
    value = world * STEP_BYTES / (ms_per_step * 1e-3) / 1e9
    e2e_value = world * STEP_BYTES / (max(e2e_ms, e2e_wall_ms) / args.steps * 1e-3) / 1e9
    per_launch_bytes = STEP_BYTES / len(sets[0])
    per_launch_s = ms_per_step * 1e-3 / len(sets[0])
    achieved = per_launch_bytes / per_launch_s / 1e9
    traffic = None
    try:
        with open(os.path.join(ROOT, "profiles", "traffic.json")) as f:
            traffic = json.load(f).get("dense_gemv_sweep_bytes_per_launch")
    except Exception:
        pass

    from oracle import binding as ob
    ob.build()
    threads = ob.host_threads()
    cpu = cpu_sample(threads)

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warm,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "code_bytes_per_step": STEP_BYTES, "linears_per_step": len(sets[0]),
                   "l2": f"weights rotate over {copies} copies ({copies * STEP_BYTES / 1e6:.0f} MB of codes > L2)",
                   "launch": launch_mode,
                   "multi_gpu": "replicas only: each rank runs the sweep on its own weight copies, no collective"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": traffic, "peak_kind": f"of {peak_kind}", "kernel": "dense_gemv_kernel (21 launches a step)"},
        "cpu_baseline": {"value": cpu["value"], "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": "one full pass of the 21-linear sweep, format.project decoding every tile per call"},
        "e2e": {"value": e2e_value, "unit": UNIT,
                "h2d_bytes_per_step": sum(i * 2 for (i, o) in SHAPES for _ in KS),
                "d2h_bytes_per_step": sum(o * 2 for (i, o) in SHAPES for _ in KS)},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "cases": cases,
    }
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cases", action="store_true", help="skip the per-linear timing table")
    ap.add_argument("--eager", action="store_true", help="time eager launches instead of replaying CUDA graphs")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
