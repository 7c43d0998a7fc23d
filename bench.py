#!/usr/bin/env python
"""Benchmark of the b200 transformer's hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One step = one pass of the workload's computation over one batch of seeded synthetic input.
Rank 0 prints ONE JSON line.  Workloads:

  c2_flex16 / c2_fp32   fused elementwise + reduction microbenchmark
                        y = tanh(a*x+b)*sigmoid(c), s = sum(y, axis 1), m = max|y| over axis 1,
                        x,a,b,c of shape (8192, 16384); y is stored (into a variable), s and m are
                        returned.  Metric: algorithmic HBM GB/s of the fused kernel.

`value` is measured with the inputs already resident in HBM (CUDA events around K launches of the
compiled computation); `e2e` goes through transformer.computation()(*host_arrays) with pinned
host arrays, host->device copies and the device->host read of the results inside the timed
region.  With --gpus N every rank runs its own replica of the workload (nothing is exchanged);
the time is the max over ranks and `value` the sum of all ranks' work over that time.

`--impl reference` times the CPU restatement of the same path (oracle/, numpy, all host cores) on
a bounded sample and prints the same line with "impl": "reference".
"""
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
sys.path.insert(0, ROOT)

C2_ROWS, C2_COLS = 8192, 16384
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum per full-size launch, scaled from the ncu capture
# of a quarter-size launch (2048 rows): see profiles/ew_c2_flex16.md and profiles/ew_c2_fp32.md
NCU_TRAFFIC_BYTES = {"c2_flex16": 4 * (268457728 + 39549952), "c2_fp32": 4 * (536940544 + 107399680)}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


def c2_algorithmic_bytes(flex, rows=C2_ROWS, cols=C2_COLS):
    """4 inputs read + y written + two row results written."""
    item = 2 if flex else 4
    return (5 * rows * cols + 2 * rows) * item


# ---------------------------------------------------------------------------------------------
class ClockSampler(object):
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([c.strip() for c in line.split(",")])

    def stop(self):
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
        for s in self.samples:
            try:
                sm.append(float(s[1]))
                mx.append(float(s[2]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, s[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


# ---------------------------------------------------------------------------------------------
def build_c2(ng, flex, rows, cols):
    R = ng.make_axis(rows, name="R")
    C = ng.make_axis(cols, name="C")
    ph = [ng.placeholder([R, C]) for _ in range(4)]
    x, a, b, c = ph
    y = ng.tanh(a * x + b) * ng.sigmoid(c)
    yvar = ng.persistent_tensor([R, C])
    s = ng.sum(y, reduction_axes=[C])
    m = ng.max(ng.absolute(y), reduction_axes=[C])
    # y is materialised on the device (assigned to a persistent tensor); s and m are returned
    out = ng.sequential([ng.assign(yvar, y), s])
    return [out, m], ph


def run_b200(args, rank, world):
    import torch
    import ngraph_python_b200 as ng
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    flex = args.workload == "c2_flex16"
    rows, cols = args.rows, C2_COLS
    t = ng.transformers.allocate_transformer("b200", device_id=local, flex=flex)
    outs, params = build_c2(ng, flex, rows, cols)
    comp = t.computation(outs, *params)
    rng = np.random.RandomState(rank)
    host = []
    for _ in range(4):
        pinned = torch.empty((rows, cols), dtype=torch.float32).pin_memory()
        arr = pinned.numpy()
        arr[...] = rng.standard_normal((rows, cols)).astype(np.float32)
        host.append(arr)
    comp(*host)            # compile, first-call exponent initialisation
    comp(*host)
    stream = torch.cuda.current_stream()

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing: inputs in HBM, K launches of the compiled step --------------
    launches0 = t.kernel_launches
    for _ in range(args.warmup):
        comp.executor()
    launches_per_step = (t.kernel_launches - launches0) // max(args.warmup, 1)
    sampler = ClockSampler(local)
    barrier()
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for _ in range(args.steps):
        comp.executor()
    ev1.record(stream)
    barrier()
    dev_ms = ev0.elapsed_time(ev1)
    # ---- end to end: host arrays in, results out ---------------------------------------------
    for _ in range(max(1, min(args.warmup, 2))):
        comp(*host)
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        res = comp(*host)
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    clocks = sampler.stop()
    h2d = sum(h.nbytes for h in host)
    d2h = sum(np.asarray(r).size for r in res) * (2 if flex else 4)
    if dist is not None:
        tt = torch.tensor([dev_ms, e2e_ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        dev_ms, e2e_ms = [float(v) for v in tt.tolist()]
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return None
    alg = c2_algorithmic_bytes(flex, rows, cols)
    ms_step = dev_ms / args.steps
    gbs = world * alg / (ms_step * 1e-3) / 1e9
    peak, which = peaks()
    kernel_gbs = alg / (ms_step * 1e-3) / 1e9
    traffic = NCU_TRAFFIC_BYTES.get(args.workload)
    line = {
        "metric": "fused-EW HBM GB/s (y=tanh(a*x+b)*sigmoid(c), row sum and row maxabs)",
        "value": round(gbs, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms_step, 5), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None,
        "dtype": "flex16 (i16 mantissa storage, f32 math)" if flex else "f32",
        "data": "synthetic",
        "config": {"workload": args.workload, "shape": [rows, cols], "replicas": world,
                   "l2": "inputs (%d MB) larger than L2" % (4 * rows * cols * (2 if flex else 4) >> 20),
                   "fused_ops": 11, "y_materialised": True},
        "clocks": clocks,
        "e2e": {"value": round(world * alg / (e2e_ms / e2e_steps * 1e-3) / 1e9, 2), "unit": "GB/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                "ms_per_step": round(e2e_ms / e2e_steps, 3)},
        "gpu_launches": launches_per_step * args.steps,
        "roofline": {"bound": "hbm", "achieved": round(kernel_gbs, 1), "peak": peak,
                     "unit": "GB/s", "frac": round(kernel_gbs / peak, 4), "traffic": traffic,
                     "peak_source": which, "algorithmic_bytes_per_launch": alg},
    }
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(args.workload, budget_s=12.0)
    if dist is not None:
        dist.destroy_process_group()
    return line


# ---------------------------------------------------------------------------------------------
def _c2_cpu_block(flex, vals):
    from oracle import ew_oracle as ew
    from oracle import flex_oracle as fx
    x, a, b, c = vals
    if flex:
        decs = [fx.fit_dec(float(np.abs(v).max())) for v in vals]
        x, a, b, c = [fx.dequantize(fx.host_to_mantissa(v, d)[0], d) for v, d in zip(vals, decs)]
    tt = ew.apply("add", ew.apply("mul", a, x), b)
    y = ew.apply("mul", ew.apply("tanh", tt), ew.apply("sig", c))
    s = y.sum(axis=1)
    m = np.abs(y).max(axis=1)
    if flex:
        y = fx.quantize(y, fx.fit_dec(float(np.abs(y).max())))
    return y, s, m


def cpu_reference_run(workload, rows, steps, warmup):
    """The CPU restatement of the workload on `rows` rows, row blocks spread over all cores."""
    from concurrent.futures import ThreadPoolExecutor
    flex = workload == "c2_flex16"
    cores = os.cpu_count() or 1
    rng = np.random.RandomState(0)
    vals = [rng.standard_normal((rows, C2_COLS)).astype(np.float32) for _ in range(4)]
    blocks = np.array_split(np.arange(rows), min(cores, rows))

    def one():
        with ThreadPoolExecutor(cores) as ex:
            list(ex.map(lambda idx: _c2_cpu_block(flex, [v[idx] for v in vals]), blocks))
    for _ in range(warmup):
        one()
    t0 = time.perf_counter()
    for _ in range(steps):
        one()
    dt = (time.perf_counter() - t0) / steps
    alg = c2_algorithmic_bytes(flex, rows, C2_COLS)
    return alg / dt / 1e9, dt, cores


def cpu_baseline(workload, budget_s=12.0):
    rows = 256
    gbs, dt, cores = cpu_reference_run(workload, rows, steps=1, warmup=1)
    steps = int(max(1, min(20, budget_s / max(dt, 1e-3))))
    gbs, dt, cores = cpu_reference_run(workload, rows, steps=steps, warmup=0)
    return {"value": round(gbs, 3), "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": "%d of %d rows x %d cols, %d passes, numpy restatement (oracle/), "
                      "row blocks on %d threads" % (rows, C2_ROWS, C2_COLS, steps, cores)}


def run_reference(args, rank, world):
    if rank != 0:
        return None
    rows = 256
    gbs, dt, cores = cpu_reference_run(args.workload, rows, max(1, args.steps), max(0, args.warmup))
    flex = args.workload == "c2_flex16"
    return {
        "impl": "reference",
        "metric": "fused-EW HBM GB/s (y=tanh(a*x+b)*sigmoid(c), row sum and row maxabs)",
        "value": round(gbs, 3), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None,
        "dtype": "flex16 (i16 mantissa storage, f32 math)" if flex else "f32",
        "data": "synthetic",
        "config": {"workload": args.workload, "shape": [C2_ROWS, C2_COLS], "replicas": world},
        "cpu_baseline": {"value": round(gbs, 3), "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": "each step = %d of %d rows x %d cols through the numpy "
                                   "restatement (oracle/), row blocks on %d threads"
                                   % (rows, C2_ROWS, C2_COLS, cores)},
        "e2e": {"value": round(gbs, 3), "unit": "GB/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c2_flex16", choices=["c2_flex16", "c2_fp32"])
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--rows", type=int, default=C2_ROWS,
                    help="rows of the microbenchmark (smaller values are for profiler captures)")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if args.impl == "reference":
        line = run_reference(args, rank, world)
    else:
        line = run_b200(args, rank, world)
    if line is not None:
        print(json.dumps(line))
        sys.stdout.flush()


if __name__ == "__main__":
    main()
