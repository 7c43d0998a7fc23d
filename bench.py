#!/usr/bin/env python
"""Benchmark of the b200 transformer's hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One step = one pass of the workload's computation over one batch of seeded synthetic input.
Rank 0 prints ONE JSON line.  Workloads:

  resnet20_flex16 / resnet20_fp32 (default: resnet20_flex16)
                        ResNet-20 inference, 3x32x32 images ~N(0,1) in C,H,W,N layout, batch 256
                        per GPU, He-initialised weights from seed 0, batch norm folded into
                        biases.  Metric: images per second.  Each GPU runs a full replica on its
                        own batch; nothing is exchanged.
  gemm_flex16 / gemm_fp32  (benchmark configuration 3) C = A.B with M = N = K = --size (default 8192);
                        flex16: int16 mantissas uniform in [-32767, 32767], exponents -15 and -12,
                        C re-quantised with the exponent chosen from its measured range.
                        Metric: T(flex-)MAC-op/s = 2MNK / t; roofline on the tensor pipe.
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

    def keep_loaded(self, load, sync, want=4, limit_s=4.0):
        """The timed region of a short run can end before nvidia-smi has produced a sample: keep
        the same workload running (untimed) until there are `want` samples under load."""
        if self.proc is None:
            return
        t0 = time.perf_counter()
        while len(self.samples) < want and time.perf_counter() - t0 < limit_s:
            for _ in range(20):
                load()
            sync()

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


# ---------------------------------------------------------------------------------------------
# ResNet-20 (benchmark configuration 4): described once as a layer list, built either as a graph for the
# b200 transformer or evaluated with the numpy restatement for the CPU baseline.
RESNET_WIDTHS = (16, 32, 64)
RESNET_N = 256
# algorithmic figures per 256-image batch: 21.03 GFLOP; minimal layer I/O of the 22 convolutions
# (inputs 58 458 112 + outputs 55 574 528 + filters 270 512 elements)
RESNET_FLOP_PER_IMG = 82.1e6
RESNET_CONV_ELEMS_PER_256 = 58458112 + 55574528 + 270512


def resnet_weights(seed=0):
    """He-initialised filters (C,R,S,K) and biases for the 22 convolutions + the linear layer."""
    r = np.random.RandomState(seed)
    convs = []

    def add(cin, cout, k):
        convs.append(((r.standard_normal((cin, k, k, cout)) * np.sqrt(2.0 / (cin * k * k)))
                      .astype(np.float32), (r.standard_normal(cout) * 0.05).astype(np.float32)))
    add(3, 16, 3)
    cin = 16
    for s, w in enumerate(RESNET_WIDTHS):
        for b in range(3):
            add(cin, w, 3)
            add(w, w, 3)
            if b == 0:
                add(cin, w, 1)
            cin = w
    lin = ((r.standard_normal((10, 64)) * np.sqrt(2.0 / 64)).astype(np.float32),
           np.zeros(10, np.float32))
    return convs, lin


def build_resnet20(ng, n, weights):
    convs, lin = weights
    ax = lambda ln, nm: ng.make_axis(ln, name=nm)   # noqa: E731
    N, D, T = ax(n, "N"), ax(1, "D"), ax(1, "T")
    x = ng.placeholder([ax(3, "C3"), D, ax(32, "H0"), ax(32, "W0"), N])
    it = iter(range(len(convs)))

    def conv(inp, c_axis, stride, sp):
        i = next(it)
        f_np, b_np = convs[i]
        cin, k = f_np.shape[0], f_np.shape[1]
        Kt = ax(f_np.shape[3], "K%d" % i)
        f = ng.variable([inp.axes[0], T, ax(k, "R%d" % i), ax(k, "S%d" % i), Kt],
                        initial_value=f_np.reshape(cin, 1, k, k, -1))
        b = ng.variable([c_axis], initial_value=b_np)
        cp = dict(pad_d=0, pad_h=k // 2, pad_w=k // 2, str_d=1, str_h=stride, str_w=stride,
                  dil_d=1, dil_h=1, dil_w=1)
        o = ng.convolution(cp, inp, f, axes=[Kt, ax(1, "M%d" % i), sp[0], sp[1], N])
        return ng.cast_axes(o, [c_axis, D, sp[0], sp[1], N]) + b
    size = 32
    sp = (ax(size, "H32"), ax(size, "W32"))
    cur = ng.maximum(conv(x, ax(16, "C16"), 1, sp), 0.0)
    for s, w in enumerate(RESNET_WIDTHS):
        c_axis = ax(w, "C%d" % w)
        for b in range(3):
            stride = 2 if (b == 0 and s > 0) else 1
            if stride == 2:
                size //= 2
                sp = (ax(size, "H%d" % size), ax(size, "W%d" % size))
            y = ng.maximum(conv(cur, c_axis, stride, sp), 0.0)
            y = conv(y, c_axis, 1, sp)
            shortcut = conv(cur, c_axis, stride, sp) if b == 0 else cur
            cur = ng.maximum(y + shortcut, 0.0)
    pool = dict(op="avg", J=1, T=1, R=size, S=size, pad_c=0, pad_d=0, pad_h=0, pad_w=0,
                str_c=1, str_d=1, str_h=1, str_w=1)
    pooled = ng.pooling(pool, cur, axes=[cur.axes[0], D, ax(1, "PP"), ax(1, "QQ"), N])
    Y = ax(10, "Y")
    w = ng.variable([Y, cur.axes[0]], initial_value=lin[0])
    by = ng.variable([Y], initial_value=lin[1])
    logits = ng.dot(w, pooled) + by
    e = ng.exp(logits - ng.max(logits, reduction_axes=[Y]))
    return [e / ng.sum(e, reduction_axes=[Y])], [x]


def resnet20_numpy(x, weights):
    """The same network with the numpy restatement (oracle/conv_oracle.py); x: (3, 32, 32, n)."""
    from oracle import conv_oracle as co
    convs, lin = weights
    it = iter(convs)

    def conv(inp, stride):
        f, b = next(it)
        k = f.shape[1]
        return co.conv_fprop(inp, f, (k // 2, k // 2), (stride, stride)) + b[:, None, None, None]
    cur = np.maximum(conv(x, 1), 0)
    for s in range(3):
        for b in range(3):
            stride = 2 if (b == 0 and s > 0) else 1
            y = np.maximum(conv(cur, stride), 0)
            y = conv(y, 1)
            shortcut = conv(cur, stride) if b == 0 else cur
            cur = np.maximum(y + shortcut, 0)
    pooled = co.pool_avg_fprop(cur, cur.shape[1:3])[:, 0, 0, :]
    logits = lin[0] @ pooled + lin[1][:, None]
    e = np.exp(logits - logits.max(axis=0))
    return e / e.sum(axis=0)


def run_resnet(args, rank, world, torch, dist, local):
    import ngraph_python_b200 as ng
    flex = args.workload == "resnet20_flex16"
    n = args.batch
    weights = resnet_weights(0)
    t = ng.transformers.allocate_transformer("b200", device_id=local, flex=flex)
    outs, params = build_resnet20(ng, n, weights)
    comp = t.computation(outs, *params)
    pinned = torch.empty((3, 1, 32, 32, n), dtype=torch.float32).pin_memory()
    host = pinned.numpy()
    host[...] = np.random.RandomState(100 + rank).standard_normal(host.shape).astype(np.float32)
    first = comp(host)[0]
    comp(host)
    if not args.no_graph:
        comp.capture()          # the step list becomes one CUDA graph launch
    stream = torch.cuda.current_stream()

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

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
    sampler.keep_loaded(comp.executor, torch.cuda.synchronize)
    # per-kind device time: events between the steps of a few instrumented passes
    kinds = {}
    passes = 5
    for _ in range(passes):
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(len(comp.steps) + 1)]
        evs[0].record(stream)
        for i, s in enumerate(comp.steps):
            t._launch_step(s)
            evs[i + 1].record(stream)
        torch.cuda.synchronize()
        for i, s in enumerate(comp.steps):
            k = kinds.setdefault(s.kind, [0.0, 0])
            k[0] += evs[i].elapsed_time(evs[i + 1])
            k[1] += 1
    # end to end
    for _ in range(2):
        comp(host)
    e2e_steps = max(1, min(args.steps, args.e2e_steps * 4))
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        res = comp(host)
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    clocks = sampler.stop()
    if dist is not None:
        tt = torch.tensor([dev_ms, e2e_ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        dev_ms, e2e_ms = [float(v) for v in tt.tolist()]
    if rank != 0:
        return None
    ms_step = dev_ms / args.steps
    peak, which = peaks()
    item = 2 if flex else 4
    # Time of all 22 convolutions of one pass.  Events between the steps need the step list
    # launched one by one, where the host's launch rate, not the kernels, sets the pace; under
    # graph replay (the timed region) the kernels run back to back.  So: the convolutions' share
    # of the launch-by-launch pass, applied to the replayed pass.
    eager_total = sum(v[0] for v in kinds.values()) / passes
    conv_ms = kinds["conv"][0] / passes
    conv_ms_source = "events between steps, launch by launch"
    if not args.no_graph and eager_total > 0 and ms_step < eager_total:
        conv_ms = ms_step * conv_ms / eager_total
        conv_ms_source = "graph-replay pass x the convolutions' share of a launch-by-launch pass"
    conv_bytes = RESNET_CONV_ELEMS_PER_256 * item * n / 256.0
    conv_gbs = conv_bytes / (conv_ms * 1e-3) / 1e9
    line = {
        "metric": "ResNet-20 %s inference img/s" % ("flex16" if flex else "fp32"),
        "value": round(world * n / (ms_step * 1e-3), 1), "unit": "img/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "flex16 (i16 mantissas, int8 hi/lo tensor-core products, i32 accumulation)"
                 if flex else "f32 (3xTF32 tensor-core products)",
        "data": "synthetic",
        "config": {"workload": args.workload, "batch_per_gpu": n, "image": [3, 32, 32],
                   "layout": "C,H,W,N", "convolutions": 22, "replicas": world,
                   "l2": "L2 flushed by the run itself: each pass streams >126 MB of "
                         "activations and operand planes",
                   "steps_per_pass": len(comp.steps), "cuda_graph": not args.no_graph},
        "clocks": clocks,
        "e2e": {"value": round(world * n / (e2e_ms / e2e_steps * 1e-3), 1), "unit": "img/s",
                "h2d_bytes_per_step": int(host.nbytes), "d2h_bytes_per_step": int(10 * n * item),
                "steps": e2e_steps, "ms_per_step": round(e2e_ms / e2e_steps, 3)},
        "gpu_launches": launches_per_step * args.steps,
        "roofline": {"bound": "hbm", "kernel": "convolution steps (gather/split + tcgen05 tile "
                     "kernel), all 22 per pass", "achieved": round(conv_gbs, 1), "peak": peak,
                     "unit": "GB/s", "frac": round(conv_gbs / peak, 4), "traffic": None,
                     "peak_source": which, "algorithmic_bytes_per_launch": int(conv_bytes),
                     "ms": round(conv_ms, 4), "ms_source": conv_ms_source},
        "step_time_ms_by_kind": {k: round(v[0] / passes, 4) for k, v in kinds.items()},
        "tensor_TOPS_algorithmic": round(RESNET_FLOP_PER_IMG * n * (4 if flex else 3)
                                         / (conv_ms * 1e-3) / 1e12, 2),
        "softmax_checksum": float(np.asarray(first).sum()),
    }
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = resnet_cpu_baseline(budget_s=12.0)
    return line


def resnet_cpu_baseline(budget_s=12.0, steps=None):
    cores = os.cpu_count() or 1
    weights = resnet_weights(0)
    n = 32
    x = np.random.RandomState(100).standard_normal((3, 32, 32, n)).astype(np.float32)
    resnet20_numpy(x, weights)
    t0 = time.perf_counter()
    resnet20_numpy(x, weights)
    dt = time.perf_counter() - t0
    reps = steps or int(max(1, min(50, budget_s / max(dt, 1e-3))))
    t0 = time.perf_counter()
    for _ in range(reps):
        resnet20_numpy(x, weights)
    dt = (time.perf_counter() - t0) / reps
    return {"value": round(n / dt, 1), "unit": "img/s", "cores": cores, "kind": "port",
            "sample": "%d passes of a %d-image batch through the numpy restatement of the "
                      "network (oracle/conv_oracle.py; numpy BLAS threads = all %d cores)"
                      % (reps, n, cores), "ms_per_step": round(dt * 1e3, 2)}


# ---- ResNet-20 data-parallel training step (global batch fixed, split over the GPUs) -----------
TRAIN_PARAM_BYTES = 1084648 + 3200      # fp32 gradients exchanged per step (weights + biases)


def run_resnet_train(args, rank, world, torch, dist, local):
    """One step = forward, backward (bprop_conv / update_conv), bucketed gradient allreduce,
    Kahan-momentum update of every parameter.  The graph is the hand-differentiated network of
    tests/golden/cases.py (pinned there against the reference CPU transformer)."""
    import ngraph_python_b200 as ng
    from ngraph_python_b200.comm import TorchDistComm, SingleProcessComm
    from tests.golden import cases
    flex = args.workload == "resnet20_train_flex16"
    gn = args.global_batch
    if gn % world or (gn // world) % 128:
        raise SystemExit("global batch must give every GPU a multiple of 128 images")
    n = gn // world
    comm = TorchDistComm() if dist is not None else SingleProcessComm()
    t = ng.transformers.allocate_transformer("b200", device_id=local, flex=flex, comm=comm,
                                             bucket_bytes=args.bucket_bytes)
    outs, params, vals = cases.resnet_train_step(ng, global_n=gn, shard=(rank, world), hw=32,
                                                 blocks=3, lr=0.002)
    comp = t.computation(outs[:1], *params)
    host = []
    for v in vals:
        pinned = torch.empty(v.shape, dtype=torch.float32).pin_memory()
        pinned.numpy()[...] = v
        host.append(pinned.numpy())
    losses = [float(comp(*host)[0]) for _ in range(3)]
    graphed = False
    if not args.no_graph:
        comp.capture()          # graphs between the NCCL exchanges (one graph on a single GPU)
        graphed = True
    stream = torch.cuda.current_stream()

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def step_resident():
        # inputs already on the device: exponent management, the step list, statistics read-back
        t._begin_call(comp)
        comp.executor()
        t._end_call(comp)

    launches0 = t.kernel_launches
    for _ in range(args.warmup):
        step_resident()
    launches_per_step = (t.kernel_launches - launches0) // max(args.warmup, 1)
    sampler = ClockSampler(local)
    barrier()
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for _ in range(args.steps):
        step_resident()
    ev1.record(stream)
    barrier()
    dev_ms = ev0.elapsed_time(ev1)
    sampler.keep_loaded(step_resident, torch.cuda.synchronize)
    kinds = {}
    passes = 3
    for _ in range(passes):
        t._begin_call(comp)
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(len(comp.steps) + 1)]
        evs[0].record(stream)
        for i, s in enumerate(comp.steps):
            t._launch_step(s)
            evs[i + 1].record(stream)
        t._end_call(comp)
        for i, s in enumerate(comp.steps):
            k = kinds.setdefault(s.kind, [0.0, 0])
            k[0] += evs[i].elapsed_time(evs[i + 1])
            k[1] += 1
    e2e_steps = max(1, min(args.steps, args.e2e_steps * 2))
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        last = comp(*host)
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    clocks = sampler.stop()
    alone_ms = nocomm_ms = 0.0
    exchanged = []
    if dist is not None and t._allreduce is not None:
        # How much of the exchange the step hides.  (1) what one step exchanges, (2) the same
        # collectives alone, back to back, (3) the step with the collectives left out; exposed
        # time = step - step without exchange.  Done last: (3) lets the replicas drift apart.
        ar, real = t._allreduce, t._allreduce.comm

        class Spy(object):
            rank, size = real.rank, real.size

            def all_reduce_async(self, flat, reduce_func="sum"):
                exchanged.append(int(flat.numel()))
                return real.all_reduce_async(flat, reduce_func)
        ar.comm = Spy()
        step_resident()
        torch.cuda.synchronize()
        per_step = list(exchanged)
        bufs = [torch.zeros(c, dtype=torch.float32, device="cuda") for c in per_step]
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for timed in (False, True):
            barrier()
            a0.record(stream)
            for _ in range(20 if timed else 3):
                for b in bufs:
                    dist.all_reduce(b)
            a1.record(stream)
            barrier()
        alone_ms = a0.elapsed_time(a1) / 20
        ar.comm = SingleProcessComm()
        for timed in (False, True):
            barrier()
            a0.record(stream)
            for _ in range(args.steps if timed else 3):
                step_resident()
            a1.record(stream)
            barrier()
        nocomm_ms = a0.elapsed_time(a1) / args.steps
        ar.comm = real
        exchanged = per_step
    if dist is not None:
        tt = torch.tensor([dev_ms, e2e_ms, alone_ms, nocomm_ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        dev_ms, e2e_ms, alone_ms, nocomm_ms = [float(v) for v in tt.tolist()]
    if rank != 0:
        return None
    ms_step = dev_ms / args.steps
    conv_ms = sum(kinds[k][0] for k in ("conv", "conv_bprop", "conv_update") if k in kinds) / passes
    tpeak, which = tensor_peak()
    tpeak = tpeak * 2 if flex else tpeak / 2
    tops = 3 * RESNET_FLOP_PER_IMG * n * (4 if flex else 3) / (conv_ms * 1e-3) / 1e12
    buckets = len(t._allreduce.plan.buckets) if t._allreduce is not None else 0
    line = {
        "metric": "ResNet-20 %s data-parallel training img/s" % ("flex16" if flex else "fp32"),
        "value": round(gn / (ms_step * 1e-3), 1), "unit": "img/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 4),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "flex16 (i16 mantissas, int8 hi/lo tensor-core products, i32 accumulation)"
                 if flex else "f32 (3xTF32 tensor-core products)",
        "data": "synthetic",
        "config": {"workload": args.workload, "global_batch": gn, "batch_per_gpu": n,
                   "image": [3, 32, 32], "layout": "C,H,W,N", "optimizer": "momentum 0.9 + Kahan",
                   "parallelism": "dp%d" % world, "allreduce_buckets": buckets,
                   "bucket_bytes": args.bucket_bytes, "steps_per_pass": len(comp.steps),
                   "cuda_graph": graphed,
                   "l2": "each step streams >126 MB of activations, gradients and operand planes"},
        "clocks": clocks,
        "e2e": {"value": round(gn / (e2e_ms / e2e_steps * 1e-3), 1), "unit": "img/s",
                "h2d_bytes_per_step": int(sum(h.nbytes for h in host)), "d2h_bytes_per_step": 4,
                "steps": e2e_steps, "ms_per_step": round(e2e_ms / e2e_steps, 3)},
        "gpu_launches": launches_per_step * args.steps,
        "roofline": {"bound": "tensor", "kernel": "convolution fprop + bprop + update steps",
                     "achieved": round(tops, 2), "peak": round(tpeak, 1),
                     "unit": "TOPS (int8)" if flex else "TFLOP/s (tf32)",
                     "frac": round(tops / tpeak, 4), "traffic": None,
                     "peak_source": which + (" bf16 x 2 as int8 stand-in" if flex else
                                             " bf16 / 2 as tf32 stand-in"),
                     "ms": round(conv_ms, 4)},
        "step_time_ms_by_kind": {k: round(v[0] / passes, 4) for k, v in kinds.items()},
        "allreduce_algorithmic_bytes_per_gpu": int(2 * (world - 1) / world * TRAIN_PARAM_BYTES),
        "loss_first_steps": [round(v, 5) for v in losses], "loss_last": round(float(last[0]), 5),
    }
    if exchanged:
        exposed = max(0.0, ms_step - nocomm_ms)
        line["allreduce"] = {
            "collectives_per_step": len(exchanged), "bytes_per_step": int(4 * sum(exchanged)),
            "alone_ms": round(alone_ms, 4), "step_without_exchange_ms": round(nocomm_ms, 4),
            "exposed_ms": round(exposed, 4),
            "overlap_frac": round(min(1.0, max(0.0, 1.0 - exposed / alone_ms)), 3) if alone_ms > 0 else None}
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = train_cpu_baseline()
    return line


def train_cpu_baseline(steps=1):
    """The same training graph evaluated with numpy (tests/mirror_interp.py over oracle/)."""
    import ngraph_python_b200 as ng
    from tests.golden import cases
    from tests import mirror_interp
    gn = 32
    outs, params, vals = cases.resnet_train_step(ng, global_n=gn, hw=32, blocks=3, lr=0.002)
    interp = mirror_interp.Interp()
    t0 = time.perf_counter()
    for _ in range(steps):
        interp.run(outs[:1], dict(zip(params, vals)))
    dt = (time.perf_counter() - t0) / steps
    cores = os.cpu_count() or 1
    return {"value": round(gn / dt, 2), "unit": "img/s", "cores": cores, "kind": "port",
            "sample": "%d training step(s) on a %d-image batch, numpy restatement of every op "
                      "(numpy BLAS threads = all %d cores)" % (steps, gn, cores),
            "ms_per_step": round(dt * 1e3, 1)}


def tensor_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["bf16_tflops"]), "measured"
    return 1590.0, "fallback"


def run_gemm(args, rank, world, torch, dist, local):
    import ngraph_python_b200 as ng
    flex = args.workload == "gemm_flex16"
    n = args.size
    t = ng.transformers.allocate_transformer("b200", device_id=local, flex=flex)
    M, K, N = ng.make_axis(n, name="M"), ng.make_axis(n, name="K"), ng.make_axis(n, name="N")
    a, b = ng.placeholder([M, K]), ng.placeholder([K, N])
    c = ng.dot(a, b)
    cvar = ng.persistent_tensor([M, N])
    # C stays on the device (assigned to a persistent tensor); its column maxima are returned
    out = ng.sequential([ng.assign(cvar, c), ng.max(cvar, reduction_axes=[M])])
    comp = t.computation(out, a, b)
    rng = np.random.RandomState(rank)
    host = []
    for scale in ((2.0 ** -15, 2.0 ** -12) if flex else (1.0, 1.0)):
        pinned = torch.empty((n, n), dtype=torch.float32).pin_memory()
        arr = pinned.numpy()
        if flex:
            arr[...] = rng.randint(-32767, 32768, (n, n)).astype(np.float32) * scale
        else:
            arr[...] = rng.standard_normal((n, n)).astype(np.float32)
        host.append(arr)
    comp(*host)
    comp(*host)
    stream = torch.cuda.current_stream()
    gemm_step = [s for s in comp.steps if s.kind == "gemm"][0]

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
    for _ in range(args.warmup):
        t._launch_step(gemm_step)
    sampler = ClockSampler(local)
    barrier()
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for _ in range(args.steps):
        t._launch_step(gemm_step)
    ev1.record(stream)
    barrier()
    dev_ms = ev0.elapsed_time(ev1)
    sampler.keep_loaded(lambda: t._launch_step(gemm_step), torch.cuda.synchronize)
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    comp(*host)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        res = comp(*host)
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    clocks = sampler.stop()
    if dist is not None:
        tt = torch.tensor([dev_ms, e2e_ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        dev_ms, e2e_ms = [float(v) for v in tt.tolist()]
    if rank != 0:
        return None
    ms_step = dev_ms / args.steps
    ops = 2.0 * n * n * n
    bf16, which = tensor_peak()
    # flex16: four int8 products per MAC; int8 peak is not measured on this pool, 2 x the
    # measured bf16 figure stands in for it (datasheet: 4500 TOPS)
    tensor_ops = (4 if flex else 3) * ops
    peak = (2 * bf16) if flex else bf16 / 2
    achieved = tensor_ops / (ms_step * 1e-3) / 1e12
    line = {
        "metric": "%s GEMM T%sMAC-op/s (2MNK/t), M=N=K=%d" % ("flex16" if flex else "fp32",
                                                              "flex-" if flex else "", n),
        "value": round(world * ops / (ms_step * 1e-3) / 1e12, 2), "unit": "Tops/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None,
        "dtype": "flex16 (int8 hi/lo tensor-core products, i32 accumulation)" if flex
                 else "f32 (3xTF32)",
        "data": "synthetic",
        "config": {"workload": args.workload, "M": n, "N": n, "K": n, "replicas": world,
                   "l2": "operand planes (%d MB) larger than L2" % (4 * n * n * (1 if flex else 4) >> 20)
                         if n >= 8192 else "operands fit in L2 at this size",
                   "includes": "operand split pre-pass + tensor-core kernel"},
        "clocks": clocks,
        "e2e": {"value": round(world * ops / (e2e_ms / e2e_steps * 1e-3) / 1e12, 3),
                "unit": "Tops/s", "h2d_bytes_per_step": int(sum(h.nbytes for h in host)),
                "d2h_bytes_per_step": int(n * (2 if flex else 4)), "steps": e2e_steps,
                "ms_per_step": round(e2e_ms / e2e_steps, 3)},
        "gpu_launches": gemm_step.launches * args.steps,
        "roofline": {"bound": "tensor", "achieved": round(achieved, 1), "peak": round(peak, 1),
                     "unit": "TOPS (int8)" if flex else "TFLOP/s (tf32)",
                     "frac": round(achieved / peak, 4), "traffic": None,
                     "peak_source": which + (" bf16 x2 as int8 stand-in" if flex
                                             else " bf16 / 2 as tf32 stand-in"),
                     "algorithmic_ops_per_launch": tensor_ops},
    }
    return line


def run_b200(args, rank, world):
    import torch
    import ngraph_python_b200 as ng
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if args.workload.startswith("gemm"):
        line = run_gemm(args, rank, world, torch, dist, local)
        if dist is not None:
            dist.destroy_process_group()
        return line
    if args.workload.startswith("resnet20_train"):
        line = run_resnet_train(args, rank, world, torch, dist, local)
        if dist is not None:
            dist.destroy_process_group()
        return line
    if args.workload.startswith("resnet20"):
        line = run_resnet(args, rank, world, torch, dist, local)
        if dist is not None:
            dist.destroy_process_group()
        return line
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
    sampler.keep_loaded(comp.executor, torch.cuda.synchronize)
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
    if args.workload.startswith("gemm"):
        n = min(args.size, 2048)
        rng = np.random.RandomState(0)
        flex = args.workload == "gemm_flex16"
        a = rng.randint(-32767, 32768, (n, n)).astype(np.float64 if flex else np.float32)
        bm = rng.randint(-32767, 32768, (n, n)).astype(np.float64 if flex else np.float32)
        a @ bm
        t0 = time.perf_counter()
        for _ in range(max(1, args.steps)):
            a @ bm
        dt = (time.perf_counter() - t0) / max(1, args.steps)
        v = round(2.0 * n ** 3 / dt / 1e12, 4)
        cores = os.cpu_count() or 1
        return {"impl": "reference", "metric": "GEMM Tops/s (2MNK/t)", "value": v,
                "unit": "Tops/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f64 (exact for int16 products)" if flex else "f32",
                "data": "synthetic", "config": {"workload": args.workload, "M": n, "N": n, "K": n},
                "cpu_baseline": {"value": v, "unit": "Tops/s", "cores": cores, "kind": "port",
                                 "sample": "numpy matmul %d^3 (the reference CPU transformer's "
                                           "Dot is np.dot), %d BLAS threads" % (n, cores)},
                "e2e": {"value": v, "unit": "Tops/s", "h2d_bytes_per_step": 0,
                        "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    if args.workload.startswith("resnet20_train"):
        flex = args.workload == "resnet20_train_flex16"
        b = train_cpu_baseline(steps=max(1, min(args.steps, 3)))
        return {
            "impl": "reference",
            "metric": "ResNet-20 %s data-parallel training img/s" % ("flex16" if flex else "fp32"),
            "value": b["value"], "unit": "img/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": b["ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32 (numpy)", "data": "synthetic",
            "config": {"workload": args.workload, "global_batch": args.global_batch,
                       "image": [3, 32, 32], "layout": "C,H,W,N"},
            "cpu_baseline": b,
            "e2e": {"value": b["value"], "unit": "img/s", "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
        }
    if args.workload.startswith("resnet20"):
        flex = args.workload == "resnet20_flex16"
        b = resnet_cpu_baseline(steps=max(1, args.steps))
        return {
            "impl": "reference",
            "metric": "ResNet-20 %s inference img/s" % ("flex16" if flex else "fp32"),
            "value": b["value"], "unit": "img/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": b["ms_per_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32 (numpy)", "data": "synthetic",
            "config": {"workload": args.workload, "batch_per_gpu": RESNET_N, "image": [3, 32, 32],
                       "layout": "C,H,W,N", "convolutions": 22, "replicas": world},
            "cpu_baseline": b,
            "e2e": {"value": b["value"], "unit": "img/s", "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
        }
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
    ap.add_argument("--workload", default="resnet20_flex16",
                    choices=["resnet20_flex16", "resnet20_fp32", "c2_flex16", "c2_fp32",
                             "gemm_flex16", "gemm_fp32", "resnet20_train_flex16",
                             "resnet20_train_fp32"])
    ap.add_argument("--global-batch", type=int, default=1024,
                    help="images per training step over all GPUs (training workloads)")
    ap.add_argument("--bucket-bytes", type=int, default=25 * 1024 * 1024,
                    help="allreduce bucket size (training workloads)")
    ap.add_argument("--size", type=int, default=8192, help="M = N = K of the GEMM workloads")
    ap.add_argument("--batch", type=int, default=RESNET_N, help="images per GPU (ResNet-20)")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--rows", type=int, default=C2_ROWS,
                    help="rows of the microbenchmark (smaller values are for profiler captures)")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch kernel by kernel instead of replaying a CUDA graph")
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
