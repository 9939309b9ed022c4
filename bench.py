#!/usr/bin/env python
"""Bench of the EXL3 projection hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--quick] [--eager] [--dense-split S] [--case NAME --rows R]

Headline workload (config 2, decode rows): the dense trunk sweep, shapes 2048x2048, 2048x6144 and
6144x2048 at K in {1,2,3,4,5,6,8} bits, one f16 activation row each: 21 linears a step, 106.4 MB of trellis code bytes.
Metric: code-byte GB/s = trellis bytes read per step / step time (the reference's byte convention: code bytes only,
src/core/gpu_test.zig:136). Weights rotate over three copies (319 MB > L2), so every step streams its codes from HBM.
A step is ONE stream of 21 launches replayed from a CUDA graph (a dependent chain's semantics; each launch may prefetch
its weights while its predecessor finishes, nothing else overlaps).

The JSON line also carries: `e2e` (the same step through the quant-plugin table with HOST arrays: copy in, run, copy
out, every call), `roofline`, `cpu_baseline` (the oracle's format.project on the host cores, all threads and one), `submetrics`
(the other two parts of the metric: us per MoE layer at decode rows on config 3, prefill TFLOP/s on configs 2 and 4
shapes, per-call and on a kept W_hat), `cases` (every linear of the sweep), `rows_2048x6144_K4` (config 2's other row counts)
and `concurrent` (the 21 independent linears as parallel graph branches: what the device sustains when nothing orders them).
Optional measurements that fail are reported in place and never void the line.

At N > 1 (torchrun) every rank runs the sweep on its own weight copies (replicas, no collective) and `submetrics.sharded`
adds the two sharded paths: the routed layer expert-parallel and a trunk linear column-sharded.

`--impl reference` times the CPU restatement of the reference's host implementation (format.project) instead.
`--quick`: headline and e2e only. `--eager`: eager launches instead of graph replay (for profilers). `--case`: one named case
run eagerly a few times (moe_decode, moe_prefill, dense_prefill, resident_prefill), printing a small JSON line of its own.
"""
from __future__ import annotations

import argparse
import datetime
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
COPIES = 3  # 3 x 106 MB of codes > the 126 MB L2


def code_bytes(in_dim: int, out_dim: int, k: int) -> int:
    return in_dim * out_dim * k // 8


STEP_BYTES = sum(code_bytes(i, o, k) for (i, o) in SHAPES for k in KS)
LINEARS = len(SHAPES) * len(KS)


def measured_peaks() -> dict:
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return {"hbm": float(d["hbm_gbs"]), "tf": float(d["bf16_tflops"]), "kind": "of measured"}
    except Exception:
        return {"hbm": 6650.0, "tf": 1590.0, "kind": "of fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the GPU work runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,utilization.gpu,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "50"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.1)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                clk, mxc, util = float(parts[1]), float(parts[2]), float(parts[3])
            except ValueError:
                continue
            mx.append(mxc)
            if util > 0:  # samples taken while kernels were running
                sm.append(clk)
            for name, val in zip(names, parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples_under_load": len(sm), "samples": len(mx), "reasons": sorted(reasons)}


def host_operands(copy: int):
    """The sweep's 21 linears for weight copy `copy` as numpy arrays (seeded uniform codes, +-1 signs)."""
    from turboexl3_b200 import synth
    ops = []
    for si, (i, o) in enumerate(SHAPES):
        for k in KS:
            ops.append((i, o, 16 * k, *synth.linear(1000 * copy + 10 * si + k, i, o, 16 * k)))
    return ops


def cpu_sample(threads: int) -> dict:
    """The oracle's faithful format.project (every tile decoded per call) over one pass of the sweep, all host threads."""
    from oracle import binding as ob
    from turboexl3_b200 import synth
    ops = host_operands(0)
    xs = {i: synth.activations(7, 1, i).astype(np.float32) for i in (2048, 6144)}
    t0 = time.perf_counter()
    for (i, o, n, trellis, suh, svh) in ops:
        ob.linear_rows(xs[i], trellis, suh, svh, i, o, n, ob.MUL1, 16, threads=threads)
    dt = time.perf_counter() - t0
    return {"seconds_per_pass": dt, "value": STEP_BYTES / dt / 1e9}


def cpu_single_thread() -> dict:
    """The same oracle on ONE host thread, as the reference's own format.project runs (it is scalar and single-threaded),
    over the sweep's three K = 4 linears."""
    from oracle import binding as ob
    from turboexl3_b200 import synth
    ops = [op for op in host_operands(0) if op[2] == 64]
    xs = {i: synth.activations(7, 1, i).astype(np.float32) for i in (2048, 6144)}
    t0 = time.perf_counter()
    for (i, o, n, trellis, suh, svh) in ops:
        ob.linear_rows(xs[i], trellis, suh, svh, i, o, n, ob.MUL1, 16, threads=1)
    dt = time.perf_counter() - t0
    byts = sum(code_bytes(i, o, n // 16) for (i, o, n, _, _, _) in ops)
    return {"value": byts / dt / 1e9, "unit": UNIT, "cores": 1, "sample": "the sweep's three K = 4 linears, one row each"}



def parity_measures(got: np.ndarray, ref: np.ndarray) -> dict:
    """ref.compare, ref.compareRounded at half an f16 ulp (src/core/ref.zig:195-218) and the share of outputs whose f16 bits are
    the oracle's."""
    from oracle import binding as ob
    g, r = np.asarray(got, np.float32), np.asarray(ref, np.float32)
    return {"compare": round(ob.compare(g, r)["max_ratio"], 6), "compareRounded": round(ob.compare(g, r, 2.0 ** -11)["max_ratio"], 6),
            "bit_equal": round(float(np.mean(g.astype(np.float16) == r.astype(np.float16))), 4), "outputs": int(g.size)}


def parity_block(t3, synth, torch, sets, host_sets, x_np, x_dev, full: bool) -> dict:
    """The GPU results of this run against the CPU oracle, per config (the bars are asserted in tests/; this is the record of
    how far inside them the timed kernels are). Sampled rows for the large cases, as the reference's own large tests do."""
    from oracle import binding as ob
    ob.build()
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    out = {}
    # config 1: 4096 x 4096, K = 4, seed 0: W_hat bit for bit, and the one-row projection
    trellis, suh, svh = synth.linear(0, 4096, 4096, 64)
    what = ob.reconstruct_inner(trellis, 4096, 4096, 64, ob.MUL1)
    w_gpu = t3.dequantize(dev(trellis)).cpu().view(torch.int16).numpy().view(np.uint16)
    x1 = synth.activations(1, 1, 4096)
    y1 = t3.linear(dev(x1), dev(trellis), dev(suh), dev(svh)).float().cpu().numpy()
    out["config1_4096x4096_K4"] = {"w_hat_equal": int(np.count_nonzero(w_gpu == what)), "w_hat_total": int(what.size),
                                   **parity_measures(y1, ob.linear_rows_what(x1.astype(np.float32), what, suh, svh, 4096, 4096))}
    # config 2 at one row: the headline's 21 linears (worst case over them)
    worst = {"compare": 0.0, "compareRounded": 0.0, "bit_equal": 1.0, "outputs": 0}
    for (i, o, n, t, a, b), (_, _, _, td, ad, bd) in zip(host_sets[0], sets[0]):
        y = t3.linear(x_dev[i], td, ad, bd).float().cpu().numpy()
        m = parity_measures(y, ob.linear_rows(x_np[i].astype(np.float32), t, a, b, i, o, n, ob.MUL1, 16, threads=ob.host_threads()))
        worst = {"compare": max(worst["compare"], m["compare"]), "compareRounded": max(worst["compareRounded"], m["compareRounded"]),
                 "bit_equal": min(worst["bit_equal"], m["bit_equal"]), "outputs": worst["outputs"] + m["outputs"]}
    out["config2_sweep_rows1_worst_of_21"] = worst
    if not full:
        return out
    # config 2 past 32 rows: 2048 x 6144, K = 4, 4096 rows, seven sampled rows
    i, o = 2048, 6144
    trellis, suh, svh = synth.linear(5, i, o, 64)
    x = synth.activations(1, 4096, i)
    sample = [0, 16, 127, 128, 2047, 2500, 4095]
    y = t3.linear(dev(x), dev(trellis), dev(suh), dev(svh)).float().cpu().numpy()[sample]
    what = ob.reconstruct_inner(trellis, i, o, 64, ob.MUL1)
    out["config2_2048x6144_K4_rows4096_sampled"] = parity_measures(y, ob.linear_rows_what(x[sample].astype(np.float32), what, suh, svh, i, o))
    # configs 3 and 4: the routed layer (hidden 2048, 512 experts x 512, top-10, K = 3) at 4 rows and at 4096 tokens (sampled)
    H, I, E, topk, n = 2048, 512, 512, 10, 48
    arrs = synth.bank(3, E, H, I, n)
    bank = t3.Bank(t3.Proj(dev(arrs["gate_t"]), dev(arrs["gate_suh"]), dev(arrs["gate_svh"])),
                   t3.Proj(dev(arrs["up_t"]), dev(arrs["up_suh"]), dev(arrs["up_svh"])),
                   t3.Proj(dev(arrs["down_t"]), dev(arrs["down_suh"]), dev(arrs["down_svh"])))
    obank = ob.Bank(E, H, I, n, *[arrs[k] for k in ("gate_t", "gate_suh", "gate_svh", "up_t", "up_suh", "up_svh", "down_t", "down_suh", "down_svh")])
    for rows, sample, name in ((4, [0, 1, 2, 3], "config3_moe_rows4"), (4096, [0, 1, 2048, 4095], "config4_moe_K3_tokens4096_sampled")):
        inds, scores = synth.routing(50 + rows, rows, E, topk)
        xm = synth.activations(5, rows, H)
        ym = t3.moe(dev(xm).view(1, rows, H), bank, dev(inds).view(1, rows, topk), dev(scores).view(1, rows, topk))
        ref = ob.moe_rows(obank, xm[sample].astype(np.float32), inds[sample], scores[sample])
        out[name] = parity_measures(ym.float().cpu().numpy().reshape(rows, H)[sample], ref)
    return out


def run_reference(args) -> None:
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from oracle import binding as ob
    ob.build()
    threads = ob.host_threads()
    warm = max(0, min(args.warmup, 1))
    for _ in range(warm):
        cpu_sample(threads)
    times = [cpu_sample(threads)["seconds_per_pass"] for _ in range(max(1, min(args.steps, 5)))]
    dt = statistics.mean(times)
    value = STEP_BYTES / dt / 1e9
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": len(times), "warmup": warm, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "note": "CPU restatement of the reference's format.project (oracle port): the "
                   "reference is a Zig library and cannot be built here; steps are capped at 5 passes"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": "one full pass of the 21-linear sweep per step, every tile decoded per call"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ---- GPU side ------------------------------------------------------------------------------------------------------

def graph_of(fn):
    """fn captured into a CUDA graph after one eager run (which also does every one-time set-up)."""
    import torch
    fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    g.replay()
    torch.cuda.synchronize()
    return g


def time_us(run, reps: int) -> float:
    """Median device time of one run() in microseconds over max(reps, 20) separately timed repetitions (the reference's
    harness reports min and median over rounds, src/core/bench.zig:1-13; time_stats gives both)."""
    return time_stats(run, reps)["median"]


def time_stats(run, reps: int = 20) -> dict:
    import torch
    reps = max(reps, 20)
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
    run()  # one untimed pass
    torch.cuda.synchronize()
    for e0, e1 in evs:
        e0.record()
        run()
        e1.record()
    torch.cuda.synchronize()
    us = sorted(e0.elapsed_time(e1) * 1e3 for e0, e1 in evs)
    return {"median": statistics.median(us), "min": us[0], "reps": reps}


def moe_submetric(t3, synth, torch) -> dict:
    """Config 3: hidden 2048, 512 experts x width 512, top-10, K = 3, one shared expert; us per MoE layer."""
    H, I, E, topk, n = 2048, 512, 512, 10, 48
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    mk = lambda arrs: t3.Bank(t3.Proj(dev(arrs["gate_t"]), dev(arrs["gate_suh"]), dev(arrs["gate_svh"])),
                              t3.Proj(dev(arrs["up_t"]), dev(arrs["up_suh"]), dev(arrs["up_svh"])),
                              t3.Proj(dev(arrs["down_t"]), dev(arrs["down_suh"]), dev(arrs["down_svh"])))
    bank, shared_bank = mk(synth.bank(3, E, H, I, n)), mk(synth.bank(4, 1, H, I, n))
    out = {}
    for rows in (1, 4, 16, 32):
        calls, distinct = [], []
        for c in range(8):  # eight routings a replay: fresh experts each call, codes from HBM (604 MB bank > L2)
            inds, scores = synth.routing(50 + c + 10 * rows, rows, E, topk)
            distinct.append(len(np.unique(inds)))
            gate = (1.0 / (1.0 + np.exp(-np.random.default_rng(c).standard_normal((rows, 1))))).astype(np.float32)
            calls.append((dev(synth.activations(c, rows, H)).view(1, rows, H), dev(inds).view(1, rows, topk),
                          dev(scores).view(1, rows, topk), dev(np.zeros((rows, 1), np.int32)).view(1, rows, 1),
                          dev(gate).view(1, rows, 1)))

        side = torch.cuda.Stream()

        def layer_burst():
            # the shared expert runs on a second stream beside the routed experts; only the routed call's last launch
            # (the merge, which adds the shared output) waits for it
            main = torch.cuda.current_stream()
            for (x, i_, s_, z_, g_) in calls:
                side.wait_stream(main)
                with torch.cuda.stream(side):
                    sh = t3.moe(x, shared_bank, z_, g_)
                    ready = torch.cuda.Event()
                    ready.record(side)
                t3.moe_with_shared(x, bank, i_, s_, t3.Decode.mul1, sh, shared_ready=ready)
                main.wait_stream(side)

        g = graph_of(layer_burst)
        st = time_stats(g.replay, 20)
        us = st["median"] / len(calls)
        byts = (float(np.mean(distinct)) + 1.0) * 3 * H * I * 3 / 8
        out[f"rows{rows}"] = {"us_per_layer": round(us, 2), "us_per_layer_min": round(st["min"] / len(calls), 2),
                              "distinct_experts": float(np.mean(distinct)), "code_GBps": round(byts / us / 1e3, 1), "reps": st["reps"]}
    return out


def prefill_submetric(t3, synth, torch) -> dict:
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    out = {}
    for (i, o, k, rows) in [(2048, 6144, 4, 4096), (2048, 2048, 4, 4096), (6144, 2048, 4, 512)]:
        w = tuple(dev(a) for a in synth.linear(5, i, o, 16 * k))
        x = dev(synth.activations(1, rows, i))
        t3.linear(x, *w)
        st = time_stats(lambda: t3.linear(x, *w), 20)
        us = st["median"]
        out[f"dense_{i}x{o}_K{k}_rows{rows}"] = {"us": round(us, 1), "us_min": round(st["min"], 1),
                                                 "TFLOPS": round(2.0 * rows * i * o / us / 1e6, 1), "reps": st["reps"]}
        if rows >= 4096:  # the same call on a kept W_hat (the resident trunk: 2 bytes a weight held, nothing decoded)
            w_t = t3.resident_build(w[0])
            t3.linear_resident(x, w_t, w[1], w[2])
            st = time_stats(lambda: t3.linear_resident(x, w_t, w[1], w[2]), 20)
            us = st["median"]
            out[f"resident_{i}x{o}_rows{rows}"] = {"us": round(us, 1), "us_min": round(st["min"], 1),
                                                   "TFLOPS": round(2.0 * rows * i * o / us / 1e6, 1), "reps": st["reps"]}
    # few prefill rows (33..256): K cut into slices a CTA each; eight calls a graph replay (a call is shorter than its launch)
    for (i, o, k, rows) in [(6144, 2048, 4, 128), (2048, 6144, 4, 128)]:
        w = tuple(dev(a) for a in synth.linear(5, i, o, 16 * k))
        x = dev(synth.activations(1, rows, i))
        g = graph_of(lambda: [t3.linear(x, *w) for _ in range(8)])
        st = time_stats(g.replay, 20)
        us = st["median"] / 8
        out[f"dense_{i}x{o}_K{k}_rows{rows}"] = {"us": round(us, 1), "us_min": round(st["min"] / 8, 1),
                                                 "TFLOPS": round(2.0 * rows * i * o / us / 1e6, 1), "reps": st["reps"]}
    H, I, E, topk, n = 2048, 512, 512, 10, 48
    arrs = synth.bank(3, E, H, I, n)
    bank = t3.Bank(t3.Proj(dev(arrs["gate_t"]), dev(arrs["gate_suh"]), dev(arrs["gate_svh"])),
                   t3.Proj(dev(arrs["up_t"]), dev(arrs["up_suh"]), dev(arrs["up_svh"])),
                   t3.Proj(dev(arrs["down_t"]), dev(arrs["down_suh"]), dev(arrs["down_svh"])))
    for rows in (4096, 16384):
        inds, scores = synth.routing(77, rows, E, topk)
        x = dev(synth.activations(5, rows, H)).view(1, rows, H)
        di, ds = dev(inds).view(1, rows, topk), dev(scores).view(1, rows, topk)
        t3.moe(x, bank, di, ds)
        st = time_stats(lambda: t3.moe(x, bank, di, ds), 20)
        us = st["median"]
        out[f"moe_config4_K3_tokens{rows}"] = {"us": round(us, 1), "us_min": round(st["min"], 1),
                                               "TFLOPS": round(2.0 * rows * topk * 3 * H * I / us / 1e6, 1), "reps": st["reps"]}
    return out


def device_bank(t3, synth, torch, seed: int, experts: int, hidden: int, inter: int, n: int):
    """A routed bank whose code words are drawn on the device (uniform halfwords; the host generator would take minutes at
    config 5's size) with synth.bank's scale vectors."""
    gen = torch.Generator(device="cuda").manual_seed(seed)
    rng = np.random.default_rng(seed)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    projs = []
    for i, o in ((hidden, inter), (hidden, inter), (inter, hidden)):
        projs.append(t3.Proj(torch.randint(-32768, 32768, (experts, i // 16, o // 16, n), dtype=torch.int16, device="cuda", generator=gen),
                             dev(synth.signs(rng, (experts, i))), dev(synth.signs(rng, (experts, o), synth.pow2_inv_sqrt(i)))))
    return t3.Bank(*projs)


def sharded_submetric(t3, synth, torch, dist, rank: int, world: int) -> dict:
    """The two sharded paths (every rank calls this; at one GPU the same code runs as a world of one, so the per-N values
    compare): the routed layer expert-parallel at a fixed number of tokens a rank — config 4's geometry at K = 3 and 4096
    tokens, config 5's (hidden 7168, 256 experts x 2048, top-8, K = 4) at 8192 tokens — and config 5's q_b projection
    column-sharded, gathered in full and left sharded. Device time, median of the
    repetitions, max over ranks."""
    from turboexl3_b200 import parallel as par
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()

    def timed(fn, reps):
        fn()
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([time_stats(fn, reps)["median"]], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    out = {}
    for (name, H, I, E, topk, n, rows, kind, reps) in (("ep_moe_config4_K3", 2048, 512, 512, 10, 48, 4096, "softmax", 20),
                                                       ("ep_moe_config5_K4", 7168, 2048, 256, 8, 64, 8192, "sigmoid", 5)):
        local = device_bank(t3, synth, torch, 100 + rank, E // world, H, I, n)  # this rank's experts only
        inds, scores = synth.routing(200 + rank, rows, E, topk, kind=kind)
        x, di, ds = dev(synth.activations(300 + rank, rows, H)), dev(inds), dev(scores)
        us = timed(lambda: par.ep_moe_cuda(x, local, di, ds, E, t3.Decode.mul1), reps)
        out[name] = {"tokens_per_rank": rows, "us_per_layer": round(us, 1), "tokens_per_s": round(world * rows / us * 1e6),
                     "TFLOPS": round(world * 2.0 * rows * topk * 3 * H * I / us / 1e6, 1), "scaling": "weak",
                     "exchange": "all_to_all_single: each token row once to every rank that owns one of its experts, "
                                 "per-slot v rows back; merge at the home rank in slot order"}
        del local, x
        torch.cuda.empty_cache()
    in_dim, out_dim = 1536, 24576
    trellis, suh, svh = synth.linear(400, in_dim, out_dim, 64)
    t_sh, svh_sh = par.shard_columns(dev(trellis), dev(svh), rank, world)
    suh_d = dev(suh)
    for r in (1, 4096):
        xr = dev(synth.activations(401 + r, r, in_dim))
        res = {}
        for label, kw in (("gathered", {}), ("left_sharded", {"gather": "none"})):
            res[label + "_us"] = round(timed(lambda: par.column_sharded_linear(xr, t_sh, suh_d, svh_sh, out_dim, t3.Decode.mul1, **kw), 20), 1)
        best = res["gathered_us"]
        out[f"column_sharded_q_b_1536x24576_K4_rows{r}"] = {
            **res, "TFLOPS_gathered": round(2.0 * r * in_dim * out_dim / best / 1e6, 1),
            "TFLOPS_left_sharded": round(2.0 * r * in_dim * out_dim / res["left_sharded_us"] / 1e6, 1), "scaling": "strong",
            "exchange": "all_gather_into_tensor of y column shards (none when left sharded)"}
    return out


def trunk_submetric(t3, synth, torch) -> dict:
    """Config 5's MLA trunk projections (K = 4) at one row: larger linears than the sweep's, where bytes start to
    matter. Each linear runs over enough distinct weight copies (slices of one 288 MB buffer of random codes) to stream
    from HBM, one graph of launches a shape."""
    n = 64
    pool = torch.randint(0, 2 ** 31 - 1, (288 * 1024 * 1024 // 4,), dtype=torch.int32, device="cuda").view(torch.int16)
    out = {}
    for name, i, o in (("q_a", 7168, 1536), ("q_b", 1536, 24576), ("kv_a", 7168, 640), ("kv_b", 512, 32768), ("o", 16384, 7168)):
        halfs = (i // 16) * (o // 16) * n
        copies = max(3, min(48, pool.numel() // halfs))
        ws = [pool[c * halfs:(c + 1) * halfs].view(i // 16, o // 16, n) for c in range(copies)]
        _, suh, svh = synth.linear(7, i, 128, 16)
        suh_d = torch.from_numpy(suh).cuda()
        svh_d = torch.from_numpy(np.where(np.random.default_rng(8).random(o) < 0.5, -1.0, 1.0).astype(np.float16)).cuda()
        x = torch.from_numpy(synth.activations(9, 1, i)).cuda()

        def burst():
            for w in ws:
                t3.linear(x, w, suh_d, svh_d)
        g = graph_of(burst)
        st = time_stats(g.replay, 20)
        us = st["median"] / copies
        byts = i * o * n // 128
        out[f"{name}_{i}x{o}"] = {"us": round(us, 2), "us_min": round(st["min"] / copies, 2), "GBps": round(byts / us / 1e3, 1),
                                  "MB": round(byts / 1e6, 1), "reps": st["reps"]}
        if name in ("q_b", "o"):
            # what bounds it: the same launches with the codebook hash skipped, the window extraction skipped too, and
            # nothing but the code stream (the kernel's timing probes; their y is not the linear's)
            probes = {}
            try:
                for label, mode in (("no_hash_us", 1), ("no_funnel_us", 2), ("stream_only_us", 3)):
                    t3.configure(probe=mode)
                    gp = graph_of(burst)
                    probes[label] = round(time_stats(gp.replay, 20)["median"] / copies, 2)
            finally:
                t3.configure()
            out[f"{name}_{i}x{o}"]["probes"] = probes
    return out


def run_case(args) -> None:
    """One named case run eagerly a few times (for profilers): prints a small JSON line, not the bench contract's."""
    import torch

    import turboexl3_b200 as t3
    from turboexl3_b200 import synth
    torch.cuda.set_device(0)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    H, I, E, topk, n = 2048, 512, 512, 10, 48
    reps = max(1, args.steps)
    if args.case in ("moe_decode", "moe_prefill"):
        arrs = synth.bank(3, E, H, I, n)
        bank = t3.Bank(t3.Proj(dev(arrs["gate_t"]), dev(arrs["gate_suh"]), dev(arrs["gate_svh"])),
                       t3.Proj(dev(arrs["up_t"]), dev(arrs["up_suh"]), dev(arrs["up_svh"])),
                       t3.Proj(dev(arrs["down_t"]), dev(arrs["down_suh"]), dev(arrs["down_svh"])))
        rows = args.rows if args.case == "moe_decode" else max(args.rows, 4096)
        calls = []
        for c in range(4):
            inds, scores = synth.routing(50 + c, rows, E, topk)
            calls.append((dev(synth.activations(c, rows, H)).view(1, rows, H), dev(inds).view(1, rows, topk),
                          dev(scores).view(1, rows, topk)))
        run = lambda: [t3.moe(x, bank, i_, s_) for (x, i_, s_) in calls]
        per = len(calls)
    elif args.case == "dense_decode":
        # one linear at decode rows over enough weight copies (random codes) to stream from HBM: --shape INxOUTxK
        i, o, k = (int(v) for v in (args.shape or "16384x7168x4").lower().split("x"))
        halfs = (i // 16) * (o // 16) * 16 * k
        copies = max(2, min(8, int(400e6 // (2 * halfs))))
        pool = torch.randint(0, 2 ** 31 - 1, (copies * halfs // 2,), dtype=torch.int32, device="cuda").view(torch.int16)
        ws = [pool[c * halfs:(c + 1) * halfs].view(i // 16, o // 16, 16 * k) for c in range(copies)]
        _, suh, svh = synth.linear(7, i, o, 16)
        suh_d, svh_d = dev(suh), dev(svh)
        x = dev(synth.activations(9, min(max(args.rows, 1), 32), i))
        if args.probe:
            t3.configure(probe=args.probe)
        run = lambda: [t3.linear(x, w, suh_d, svh_d) for w in ws]
        per = copies
    else:
        i, o, k = (int(v) for v in (args.shape or "2048x6144x4").lower().split("x"))
        w = tuple(dev(a) for a in synth.linear(5, i, o, 16 * k))
        x = dev(synth.activations(1, max(args.rows, 33), i))
        if args.case == "resident_prefill":
            w_t = t3.resident_build(w[0])
            run = lambda: t3.linear_resident(x, w_t, w[1], w[2])
        else:
            run = lambda: t3.linear(x, *w)
        per = 1
    run()
    us = time_us(run, reps) / per
    print(json.dumps({"case": args.case, "rows": args.rows, "us_per_call": round(us, 2), "device_error": t3.device_error()}))


def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    import turboexl3_b200 as t3
    from turboexl3_b200 import synth
    from turboexl3_b200 import table as tb

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        # NCCL writes its version banner to stdout at the first communicator; keep stdout for the one JSON line
        sys.stdout.flush()
        keep = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=180))
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(keep, 1)
            os.close(keep)
    t3.lib()
    if args.dense_split:
        t3.configure(dense_split=args.dense_split)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()

    host_sets = [host_operands(c) for c in range(COPIES)]
    sets = [[(i, o, n, torch.from_numpy(t).cuda(), torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda())
             for (i, o, n, t, a, b) in ops] for ops in host_sets]
    x_np = {i: synth.activations(7, 1, i) for i in (2048, 6144)}
    x_dev = {i: torch.from_numpy(v).cuda() for i, v in x_np.items()}
    dec = t3.Decode.mul1

    def step_eager(c: int):
        for (i, o, n, t, a, b) in sets[c]:
            t3.linear(x_dev[i], t, a, b, dec)

    def step_branches(c: int):
        """The same 21 launches as independent branches of the graph (forked streams)."""
        main = torch.cuda.current_stream()
        side = [torch.cuda.Stream() for _ in range(7)]
        for s in side:
            s.wait_stream(main)
        for idx, (i, o, n, t, a, b) in enumerate(sets[c]):
            with torch.cuda.stream(side[idx % 7]):
                t3.linear(x_dev[i], t, a, b, dec)
        for s in side:
            main.wait_stream(s)

    graphs, launch_mode = [], "one stream, 21 kernel nodes replayed from a CUDA graph per step"
    if not args.eager:
        try:
            graphs = [graph_of(lambda c=c: step_eager(c)) for c in range(COPIES)]
        except Exception as exc:
            graphs, launch_mode = [], f"eager launches (graph capture failed: {type(exc).__name__})"
            torch.cuda.synchronize()
    else:
        launch_mode = "eager launches"

    def step_device(s: int):
        if graphs:
            graphs[s % COPIES].replay()
        else:
            step_eager(s % COPIES)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    warm = max(args.warmup, 3)
    for s in range(warm):
        step_device(s)
    barrier()
    launches0 = t3.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for s in range(args.steps):
        step_device(warm + s)
    ev1.record()
    barrier()
    ms = ev0.elapsed_time(ev1)
    launches = LINEARS * args.steps if graphs else t3.launch_count() - launches0

    # ---- end to end: the quant-plugin table on HOST arrays (weights resident, activations copied in and out per call)
    blk = tb.Block('{"format":"exl3","codebook":"mul1"}')
    assert blk.verdict.ok
    table_sets = []
    for ops in host_sets:
        ws = []
        for (i, o, n, t, a, b) in ops:
            v, w = blk.load_tensor(t, a, b, i)
            assert v.ok, v.why
            ws.append(w)
        table_sets.append(ws)
    import ctypes as C
    tab = tb.table()
    y_np = {o: np.empty((1, o), np.float16) for o in (2048, 6144)}
    x_arr = {i: tb.host_array(v) for i, v in x_np.items()}
    y_arr = {o: tb.host_array(v) for o, v in y_np.items()}
    stream_ptr = torch.cuda.current_stream().cuda_stream

    x_ref = {i: C.byref(v) for i, v in x_arr.items()}
    y_ref = {o: C.byref(v) for o, v in y_arr.items()}
    calls = [[(C.byref(w), x_ref[w.in_dim], y_ref[w.out_dim]) for w in ws] for ws in table_sets]
    matmul = tab.matmul

    def step_e2e(s: int):
        for (w_ref, xr, yr) in calls[s % COPIES]:
            v = matmul(w_ref, xr, stream_ptr, yr)
            if v.kind != 0:
                raise SystemExit(f"table matmul refused: {v.reason}")

    e2e_steps = max(3, min(args.steps, 20))
    for s in range(2):
        step_e2e(s)
    barrier()
    t0 = time.perf_counter()
    for s in range(e2e_steps):
        step_e2e(2 + s)
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3  # every call ends with its result on the host: wall time is the measure
    for ws in table_sets:
        for w in ws:
            tab.release(C.byref(w))
    blk.close()

    # the headline and the end-to-end figure are in: they must be clean, and they are reduced over the ranks before
    # anything optional runs, so that a failing extra cannot take the line with it
    if t3.device_error() != 0:
        raise SystemExit("a kernel reported a bounded-wait failure; the numbers are void")
    times = torch.tensor([ms / args.steps, e2e_ms / e2e_steps], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_per_step, e2e_ms_per_step = times.tolist()
    clocks = sampler.stop() if rank == 0 else None  # the samples cover the timed regions above

    def guarded(fn):
        """An optional measurement: its result, or what stopped it."""
        try:
            out = fn()
            bits = t3.device_error()
            return out if bits == 0 else {"error": f"a kernel's bounded wait ran out (bits {bits}); numbers dropped"}
        except Exception as exc:  # noqa: BLE001 - reported in the line
            return {"error": f"{type(exc).__name__}: {str(exc)[:120]}"}

    # the sharded paths first: every rank takes part, and the other ranks must not sit in a collective while rank 0 runs
    # its single-GPU extras
    sharded = None
    if not args.quick:
        if world == 1 and not dist.is_initialized():  # a world of one, so the sharded paths run the code they run at N > 1
            import socket
            with socket.socket() as sk:
                sk.bind(("127.0.0.1", 0))
                port = sk.getsockname()[1]
            keep = os.dup(1)
            os.dup2(2, 1)
            try:
                dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1,
                                        device_id=torch.device("cuda", local))
            finally:
                sys.stdout.flush()
                os.dup2(keep, 1)
                os.close(keep)
        sharded = guarded(lambda: sharded_submetric(t3, synth, torch, dist, rank, world))
    extra = {}
    if sharded is not None:
        extra.setdefault("submetrics", {})["sharded"] = sharded
    if rank == 0 and not args.quick:
        # the 21 linears with nothing ordering them
        try:
            bgraphs = [graph_of(lambda c=c: step_branches(c)) for c in range(COPIES)]
            for s in range(3):
                bgraphs[s % COPIES].replay()
            idx = [0]

            def replay_next():
                bgraphs[idx[0] % COPIES].replay()
                idx[0] += 1

            us = time_us(replay_next, 30)
            extra["concurrent"] = {"value": round(STEP_BYTES / us / 1e3, 1), "unit": UNIT, "us_per_step": round(us, 1),
                                   "what": "the step's 21 independent linears as parallel branches of one CUDA graph"}
        except Exception as exc:
            extra["concurrent"] = {"error": type(exc).__name__}
        # per-linear device time: a graph of one launch per weight copy
        def per_linear():
            cases = {}
            for idx, (i, o, n, _, _, _) in enumerate(sets[0]):
                def burst(idx=idx, i=i):
                    for c in range(COPIES):
                        t3.linear(x_dev[i], *sets[c][idx][3:], dec)
                g = graph_of(burst) if graphs else None
                us = time_us(g.replay if g is not None else burst, 10) / COPIES
                cases[f"{i}x{o}_K{n // 16}"] = {"us": round(us, 2), "GBps": round(code_bytes(i, o, n // 16) / us / 1e3, 1)}
            return cases
        extra["cases"] = guarded(per_linear)

        def per_rows():
            """config 2's other in-register row counts on one linear (2048 x 6144, K = 4): the bytes do not grow with rows"""
            idx = next(j for j, (i, o, n, _, _, _) in enumerate(sets[0]) if (i, o, n) == (2048, 6144, 64))
            out = {}
            for rows in (1, 8, 17, 32):
                xr = torch.from_numpy(synth.activations(9, rows, 2048)).cuda()

                def burst():
                    for c in range(COPIES):
                        t3.linear(xr, *sets[c][idx][3:], dec)
                g = graph_of(burst) if graphs else None
                us = time_us(g.replay if g is not None else burst, 10) / COPIES
                out[f"rows{rows}"] = {"us": round(us, 2), "GBps": round(code_bytes(2048, 6144, 4) / us / 1e3, 1)}
            return out
        extra["rows_2048x6144_K4"] = guarded(per_rows)
        extra["trunk_config5_K4_rows1"] = guarded(lambda: trunk_submetric(t3, synth, torch))
        extra.setdefault("submetrics", {}).update({"moe_layer_decode_rows_config3": guarded(lambda: moe_submetric(t3, synth, torch)),
                                                   "prefill": guarded(lambda: prefill_submetric(t3, synth, torch))})

    if rank != 0:
        if dist.is_initialized():
            dist.destroy_process_group()
        return

    extra["parity"] = guarded(lambda: parity_block(t3, synth, torch, sets, host_sets, x_np, x_dev, full=not args.quick))

    peaks = measured_peaks()
    value = world * STEP_BYTES / (ms_per_step * 1e-3) / 1e9
    achieved = (STEP_BYTES / LINEARS) / (ms_per_step * 1e-3 / LINEARS) / 1e9
    # DRAM bytes a launch of the dominant kernel moves: captured once under ncu (profiles/traffic.json), stamped with the
    # digest of the kernel sources it was captured on; a capture taken on other sources is reported as stale, not as current
    traffic, traffic_note = None, "no capture"
    try:
        from turboexl3_b200 import build as t3_build
        with open(os.path.join(ROOT, "profiles", "traffic.json")) as f:
            cap = json.load(f)
        traffic = cap.get("dense_gemv_sweep_bytes_per_launch")
        traffic_note = ("captured on these kernel sources" if cap.get("sources_digest") == t3_build.sources_digest()
                        else "captured on earlier kernel sources")
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
        "config": {"workload": WORKLOAD, "code_bytes_per_step": STEP_BYTES, "linears_per_step": LINEARS,
                   "l2": f"weights rotate over {COPIES} copies ({COPIES * STEP_BYTES / 1e6:.0f} MB of codes > L2)",
                   "launch": launch_mode,
                   "multi_gpu": "replicas only: each rank runs the sweep on its own weight copies, no collective"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm"], "traffic": traffic, "traffic_capture": traffic_note, "peak_kind": peaks["kind"],
                     "kernel": "t3_dense_gemv_<codebook>_n<n>_r8 (21 launches a step; bytes and time are the step's, per launch)"},
        "cpu_baseline": {"value": cpu["value"], "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": "one full pass of the 21-linear sweep, format.project decoding every tile per call",
                         "single_thread": cpu_single_thread()},
        "e2e": {"value": world * STEP_BYTES / (e2e_ms_per_step * 1e-3) / 1e9, "unit": UNIT,
                "h2d_bytes_per_step": sum(i * 2 for (i, o) in SHAPES for _ in KS),
                "d2h_bytes_per_step": sum(o * 2 for (i, o) in SHAPES for _ in KS),
                "api": "t3_table()->matmul on host arrays, one call a linear, result on the host when it returns"},
        "gpu_launches": int(launches),
        "clocks": clocks,
    }
    line.update(extra)
    print(json.dumps(line))
    if dist.is_initialized():
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--quick", action="store_true", help="headline and e2e only (no per-linear table, no submetrics)")
    ap.add_argument("--eager", action="store_true", help="time eager launches instead of replaying CUDA graphs")
    ap.add_argument("--dense-split", type=int, default=0, help="force the dense GEMV's K split (t3_configure; 0 = the library's choice)")
    ap.add_argument("--case", default=None, choices=["moe_decode", "moe_prefill", "dense_prefill", "resident_prefill", "dense_decode"],
                    help="run one case eagerly --steps times and exit (for profilers)")
    ap.add_argument("--rows", type=int, default=1, help="rows of --case")
    ap.add_argument("--shape", default=None, help="INxOUTxK of --case dense_decode (default 16384x7168x4) and dense_prefill / resident_prefill (default 2048x6144x4)")
    ap.add_argument("--probe", type=int, default=0, choices=[0, 1, 2, 3],
                    help="--case dense_decode with the kernel's timing probe in the served kernel's place (t3_config.probe)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.case:
        run_case(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
