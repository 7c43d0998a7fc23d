#!/usr/bin/env python
"""Benchmark of the b200 transformer's hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One step = one pass of the workload's computation over one batch of seeded synthetic input.
Rank 0 prints ONE JSON line.  Workloads:

  resnet20_flex16 / resnet20_fp32 (default: resnet20_flex16; benchmark configuration 4)
                        ResNet-20 inference, 3x32x32 images in C,H,W,N layout, batch 256 per GPU,
                        He-initialised weights from seed 0, no batch norm.  Where the reference
                        tree is at hand (B200NG_REFERENCE or oracle/_ref) the network is the
                        reference's own builder (examples/resnet/resnet.py: BuildResnet('cifar10',
                        20, False, 3, batch_norm=False)), built with the reference's `ngraph` and
                        compiled by ngraph.transformers.make_transformer_factory('b200'); the first
                        result is compared with the reference CPU transformer on the same graph and
                        input before anything is timed.  Elsewhere this package's restatement of the
                        network is used.  Metric: images per second.  Each GPU runs a full replica
                        on its own batch; nothing is exchanged.
  resnet20_train_flex16 / resnet20_train_fp32 (configuration 5)
                        one data-parallel momentum-SGD step of the same network, global batch 1024
                        split over the GPUs, bucketed NCCL gradient exchange.
  gemm_flex16 / gemm_fp32  (configuration 3) C = A.B with M = N = K = --size (default 8192).
                        Metric: T(flex-)MAC-op/s = 2MNK / t; roofline on the tensor pipe.
  c2_flex16 / c2_fp32   (configuration 2) y = tanh(a*x+b)*sigmoid(c), s = sum(y, axis 1),
                        m = max|y| over axis 1, x,a,b,c of shape (8192, 16384); y is stored.
                        Metric: algorithmic HBM GB/s of the fused kernel.

The default run carries the whole headline metric: after the ResNet-20 timed region it also runs
configurations 2 and 3 (one GPU) and the training step of configuration 5 and reports them under
`extras` (skip with --no-extras).

`value` is measured with the inputs already resident in HBM: CUDA events around K steps, each
step = the per-call exponent bookkeeping + the compiled step list (a CUDA graph) + the read-back
of statistics and status; the loop is repeated --repeats times and the median taken.  `e2e` goes
through computation(host_array) with pinned host arrays, host->device copies and the device->host
read of the results inside the timed region.  With --gpus N every rank runs its own replica; the
time is the max over ranks and `value` the sum of all ranks' work over that time.

`--impl reference` times the reference's own CPU transformer (numpy engine, all host cores) on the
same configuration and prints the same line with "impl": "reference"; without the reference tree
it falls back to the numpy restatement under oracle/ and says so (`cpu_baseline.kind`).
"""
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
sys.path.insert(0, ROOT)

C2_ROWS, C2_COLS = 8192, 16384
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
INT8_DATASHEET_TOPS = 4500.0
# dram__bytes_read.sum + dram__bytes_write.sum per full-size launch, scaled from the ncu capture
# of a quarter-size launch (2048 rows): see profiles/ew_c2_flex16.md and profiles/ew_c2_fp32.md
NCU_TRAFFIC_BYTES = {"c2_flex16": 4 * (268457728 + 39549952), "c2_fp32": 4 * (536940544 + 107399680)}
# the same two counters summed over the 22 convolution launches of one batch-256 flex16 pass
# (profiles/conv_resnet20_flex16.md).  ncu flushes the caches before every launch it measures, so
# this counts as DRAM reads what the real sequence finds in L2, and no write reaches DRAM within
# its launch: an upper bound on the reads of the timed pass, not its traffic to the byte.
NCU_CONV_TRAFFIC_BYTES = {"resnet20_flex16": 154123008}

RESNET_N = 256
# algorithmic figures per 256-image batch: 21.03 GFLOP; minimal layer I/O of the 22 convolutions
# (inputs 58 458 112 + outputs 55 574 528 + filters 270 512 elements)
RESNET_FLOP_PER_IMG = 82.1e6
RESNET_CONV_ELEMS_PER_256 = 58458112 + 55574528 + 270512
TRAIN_PARAM_BYTES = 1084648      # fp32 gradients exchanged per step (no batch norm, no biases)
REFERENCE_NETWORK = ("reference examples/resnet/resnet.py BuildResnet('cifar10', 20, False, 3, "
                     "batch_norm=False), built with the reference's ngraph")
OWN_NETWORK = "this package's restatement of ResNet-20 (reference tree absent)"
CIFAR_MEAN = np.array([113.9, 123.0, 125.3], np.float32)
CIFAR_STD = np.array([66.7, 62.1, 63.0], np.float32)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


def tensor_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["bf16_tflops"]), "measured"
    return FALLBACK_BF16_TFLOPS, "fallback"


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

    def keep_loaded(self, load, sync, want=4, limit_s=4.0, dist=None, torch=None, device="cuda"):
        """The timed region of a short run can end before nvidia-smi has produced a sample: keep
        the same workload running (untimed) until there are `want` samples under load.
        When `load` holds collectives (a data-parallel training step) every replica has to run
        it the same number of times -- a replica that stopped early would leave the others waiting
        in an exchange for ever -- so with `dist` the replicas agree after every batch of calls
        whether to go on (any of them still short of samples and within its time limit)."""
        t0 = time.perf_counter()
        while True:
            need = self.proc is not None and len(self.samples) < want and \
                time.perf_counter() - t0 < limit_s
            if dist is not None:
                flag = torch.tensor([1.0 if need else 0.0], device=device)
                dist.all_reduce(flag, op=dist.ReduceOp.MAX)
                need = bool(flag.item() > 0)
            if not need:
                return
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


class Timer(object):
    """CUDA-event timing of `repeats` loops of `steps` calls, barrier + synchronize on both sides
    of every loop, max over ranks per loop."""

    def __init__(self, torch, dist):
        self.torch, self.dist = torch, dist
        self.stream = torch.cuda.current_stream()

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.dist is not None:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def loops(self, fn, steps, repeats):
        torch = self.torch
        out = []
        for _ in range(max(1, repeats)):
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.barrier()
            ev0.record(self.stream)
            for _ in range(steps):
                fn()
            ev1.record(self.stream)
            self.barrier()
            out.append(ev0.elapsed_time(ev1))
        if self.dist is not None:
            tt = torch.tensor(out, dtype=torch.float64, device="cuda")
            self.dist.all_reduce(tt, op=self.dist.ReduceOp.MAX)
            out = [float(v) for v in tt.tolist()]
        return out

    def wall(self, fn, steps):
        """Host wall-clock around `steps` blocking calls (the end-to-end figure), max over ranks."""
        self.barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            fn()
        self.torch.cuda.synchronize()
        ms = (time.perf_counter() - t0) * 1e3
        if self.dist is not None:
            tt = self.torch.tensor([ms], dtype=self.torch.float64, device="cuda")
            self.dist.all_reduce(tt, op=self.dist.ReduceOp.MAX)
            ms = float(tt.item())
        return ms


def spread(loop_ms, steps):
    per = sorted(v / steps for v in loop_ms)
    return {"n": len(per), "median": round(statistics.median(per), 5), "min": round(per[0], 5),
            "max": round(per[-1], 5)}


# ---------------------------------------------------------------------------------------------
# the reference front end (real `ngraph` ops + the plug-in), where a tree of it is at hand
def reference_root():
    for c in (os.environ.get("B200NG_REFERENCE"), os.path.join(ROOT, "oracle", "_ref")):
        if c and os.path.isdir(os.path.join(c, "ngraph")):
            return os.path.abspath(c)
    return None


_frontend = {}


def reference_frontend():
    """(ngraph module, ngraph.transformers module) with the b200 plug-in registered, or None."""
    if "mods" in _frontend:
        return _frontend["mods"]
    root = reference_root()
    mods = None
    if root is not None:
        from ngraph_python_b200 import ngraph_compat
        ngraph_compat.install(root)
        ex = os.path.join(root, "examples", "resnet")
        if ex not in sys.path:
            sys.path.insert(0, ex)
        import contextlib
        import io
        with contextlib.redirect_stdout(io.StringIO()):      # "Could not load MKLDNN Engine ..."
            import ngraph as rng
            import ngraph.transformers as ngt
            import ngraph_python_b200.ngraph_plugin  # noqa: F401
        mods = (rng, ngt)
    _frontend["mods"] = mods
    return mods


def reference_resnet20(rng, n, train=False, lr=0.1, momentum=0.9, features=False):
    """examples/resnet/resnet.py:74-117 of the reference: CIFAR-10 ResNet-20 without batch norm.
    Returns (result op, placeholders)."""
    from resnet import BuildResnet
    from ngraph.frontends.neon import ax, Layer, GradientDescentMomentum
    ax.N.length = n
    ax.Y.length = 10
    C, H, W = rng.make_axis(3, name="C"), rng.make_axis(32, name="H"), rng.make_axis(32, name="W")
    x = rng.placeholder([C, H, W, ax.N])
    np.random.seed(0)
    model = BuildResnet('cifar10', 20, False, 3, batch_norm=False)
    if not train:
        with Layer.inference_mode_on():
            out = model(x)
            if features:
                # the pooled features that feed the linear layer (same layers, same weights): the
                # softmax of this network without batch norm is all but one-hot, the features
                # are what a parity check can bite on
                from ngraph.frontends.neon import Sequential
                return out, [x], Sequential(model.layers[:-2])(x)
            return out, [x]
    t = rng.placeholder([ax.N])
    loss = rng.cross_entropy_multi(model(x), rng.one_hot(t, axis=ax.Y))
    updates = GradientDescentMomentum(lr, momentum)(loss)
    return rng.sequential([updates, rng.mean(loss, out_axes=[])]), [x, t]


def cifar_like(seed, n):
    """Images whose preprocessed values (the reference network subtracts the CIFAR-10 channel
    means and divides by the channel deviations first) are ~N(0,1): mean + std * N(0,1)."""
    z = np.random.RandomState(seed).standard_normal((3, 32, 32, n)).astype(np.float32)
    return z * CIFAR_STD[:, None, None, None] + CIFAR_MEAN[:, None, None, None]


# ---------------------------------------------------------------------------------------------
# this package's restatement of the network, used where the reference tree is absent
RESNET_WIDTHS = (16, 32, 64)


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


def flex_tolerance(desired):
    """The reference's flex tolerance (ngraph/transformers/flexgputransform.py:80-103): atol =
    8 steps of a flex16 tensor that just holds max|desired|, rtol 1e-2."""
    m = float(np.max(np.abs(desired)))
    dec = 15 - int(np.floor(np.log2(m))) - 1 if m > 0 else 8
    while m * 2.0 ** dec > 32767:
        dec -= 1
    return 8 * 2.0 ** -dec, 1e-2


def resnet_config(workload, n, world, frontend):
    return {"workload": workload, "batch_per_gpu": n, "image": [3, 32, 32], "layout": "C,H,W,N",
            "convolutions": 22, "network": frontend}


class ResnetInference(object):
    """The compiled ResNet-20 inference computation on one GPU, through whichever front end is
    available.  `comp` is this package's Computation, `t` its B200Transformer."""

    def __init__(self, torch, local, flex, n, seed):
        self.flex, self.n = flex, n
        fe = reference_frontend()
        if fe is not None:
            rng, ngt = fe
            out, params, feat = reference_resnet20(rng, n, features=True)
            self.outer_t = ngt.make_transformer_factory("b200", device_id=local, flex=flex)()
            self.call = self.outer_t.computation(out, *params)
            self.check = self.outer_t.computation([out, feat], *params)
            self.t, self.comp = self.outer_t.impl, self.call.impl
            self.frontend = REFERENCE_NETWORK
            self.graph = ([out, feat], params)
            shape, data = (3, 32, 32, n), cifar_like(seed, n)
        else:
            import ngraph_python_b200 as ng
            self.weights = resnet_weights(0)
            self.outer_t = ng.transformers.allocate_transformer("b200", device_id=local, flex=flex)
            outs, params = build_resnet20(ng, n, self.weights)
            self.call = self.outer_t.computation(outs[0], *params)
            self.check = self.outer_t.computation([outs[0]], *params)
            self.t, self.comp = self.outer_t, self.call
            self.frontend = OWN_NETWORK
            self.graph = None
            shape = (3, 1, 32, 32, n)
            data = np.random.RandomState(seed).standard_normal(shape).astype(np.float32)
        self.pinned = torch.empty(shape, dtype=torch.float32).pin_memory()
        self.host = self.pinned.numpy()
        self.host[...] = data

    def cpu_expectation(self):
        """(expected results, what computed them) on the host cores, same graph and input: the
        softmax and, with the reference front end, the pooled features under it."""
        fe = reference_frontend()
        if fe is not None and self.graph is not None:
            _, ngt = fe
            cpu = ngt.make_transformer_factory("cpu")()
            res = cpu.computation(self.graph[0], *self.graph[1])(self.host)
            want = [np.array(r, copy=True) for r in res]
            cpu.close()
            return want, "reference CPUTransformer, same graph and input"
        want = [resnet20_numpy(self.host[:, 0], self.weights)]
        return want, "numpy restatement (oracle/conv_oracle.py), same weights and input"

    def close(self):
        self.outer_t.close()


def check_parity(got, want, flex):
    """got, want: lists [softmax (10, n), pooled features (64, ..., n) if available]."""
    report = {"ok": True}
    for name, g_, w_ in zip(("softmax", "pooled_features"), got, want):
        w_ = np.asarray(w_, dtype=np.float64)
        g_ = np.asarray(g_, dtype=np.float64).reshape(w_.shape)
        if flex:
            atol, rtol = flex_tolerance(w_)
            atol *= 4          # the expectation is the fp32 result, not a flex evaluation
        else:
            atol, rtol = 1e-5 * max(1.0, float(np.max(np.abs(w_)))), 1e-4
        ok = bool(np.all(np.abs(g_ - w_) <= atol + rtol * np.abs(w_)))
        report[name] = {"ok": ok, "max_abs_err": float(np.max(np.abs(g_ - w_))),
                        "max_abs_expected": float(np.max(np.abs(w_))), "atol": atol, "rtol": rtol}
        report["ok"] = report["ok"] and ok
    w0 = np.asarray(want[0])
    report["argmax_agreement"] = float((np.asarray(got[0]).reshape(w0.shape).argmax(axis=0)
                                        == w0.argmax(axis=0)).mean())
    return report


def run_resnet(args, rank, world, torch, dist, local):
    flex = args.workload == "resnet20_flex16"
    n = args.batch
    net = ResnetInference(torch, local, flex, n, seed=100 + rank)
    t, comp, host = net.t, net.comp, net.host
    first = [np.array(r, copy=True) for r in net.check(host)]
    parity = None
    if rank == 0:
        want, how = net.cpu_expectation()
        parity = check_parity(first, want, flex)
        parity["against"] = how
        if not parity["ok"]:
            raise SystemExit("parity check failed before timing: %s" % json.dumps(parity))
    net.call(host)
    if not args.no_graph:
        comp.capture()          # the step list becomes one CUDA graph launch
    timer = Timer(torch, dist)

    def step_resident():
        # inputs already on the device: exponent bookkeeping, the step list, statistics read-back
        t._begin_call(comp)
        comp.executor()
        t._end_call(comp)

    launches0 = t.kernel_launches
    for _ in range(args.warmup):
        step_resident()
    launches_per_step = (t.kernel_launches - launches0) // max(args.warmup, 1)
    sampler = ClockSampler(local)
    timer.barrier()
    sampler.start()
    loop_ms = timer.loops(step_resident, args.steps, args.repeats)
    sampler.keep_loaded(step_resident, torch.cuda.synchronize)
    replay_ms = timer.loops(comp.executor, args.steps, args.repeats)
    # the 22 convolution launches alone, back to back, as a CUDA graph of their own: every tensor
    # they read is still in place from the last pass
    conv_steps = [s for s in comp.steps if s.kind == "conv"]

    def convs_only():
        for s in conv_steps:
            t._launch_step(s)
    conv_fn, conv_src = convs_only, "CUDA events around the 22 convolution steps launched one by one"
    if not args.no_graph:
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            convs_only()
        conv_fn = g.replay
        conv_src = "CUDA events around a replayed graph of the 22 convolution steps alone"
    conv_loops = timer.loops(conv_fn, args.steps, args.repeats)
    # end to end
    for _ in range(2):
        net.call(host)
    e2e_steps = max(1, min(args.steps, args.e2e_steps * 4))
    e2e_ms = timer.wall(lambda: net.call(host), e2e_steps)
    clocks = sampler.stop()
    if rank != 0:
        net.close()
        return None
    ms_step = statistics.median(loop_ms) / args.steps
    replay_step = statistics.median(replay_ms) / args.steps
    conv_ms = statistics.median(conv_loops) / args.steps
    peak, which = peaks()
    item = 2 if flex else 4
    conv_bytes = RESNET_CONV_ELEMS_PER_256 * item * n / 256.0
    conv_gbs = conv_bytes / (conv_ms * 1e-3) / 1e9
    cfg = resnet_config(args.workload, n, world, net.frontend)
    cfg.update({"replicas": world,
                "transformer": "ngraph.transformers.make_transformer_factory('b200') (plug-in)"
                               if net.graph is not None else "ngraph_python_b200.transformers",
                "l2": "L2 flushed by the run itself: each pass streams >126 MB of activations and "
                      "operand planes",
                "steps_per_pass": len(comp.steps), "cuda_graph": not args.no_graph,
                "value_includes": "per-call exponent bookkeeping, graph replay, statistics and "
                                  "status read-back with one stream synchronisation"})
    traffic = NCU_CONV_TRAFFIC_BYTES.get(args.workload)
    line = {
        "metric": "ResNet-20 %s inference img/s" % ("flex16" if flex else "fp32"),
        "value": round(world * n / (ms_step * 1e-3), 1), "unit": "img/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "flex16 (i16 mantissas, int8 hi/lo tensor-core products, i32 accumulation)"
                 if flex else "f32 (3xTF32 tensor-core products)",
        "data": "synthetic",
        "config": cfg,
        "clocks": clocks,
        "repeats": spread(loop_ms, args.steps),
        "graph_replay_only": {"ms_per_step": round(replay_step, 4),
                              "img_s": round(world * n / (replay_step * 1e-3), 1),
                              "what": "the captured step list alone, no exponent bookkeeping or "
                                      "read-back between replays"},
        "e2e": {"value": round(world * n / (e2e_ms / e2e_steps * 1e-3), 1), "unit": "img/s",
                "h2d_bytes_per_step": int(host.nbytes), "d2h_bytes_per_step": int(10 * n * item),
                "steps": e2e_steps, "ms_per_step": round(e2e_ms / e2e_steps, 3)},
        "gpu_launches": launches_per_step * args.steps,
        "roofline": {"bound": "hbm", "kernel": "the 22 convolution steps of a pass (tcgen05 tile "
                     "kernel with fused tails)" if flex else "the 22 convolution steps of a pass",
                     "achieved": round(conv_gbs, 1), "peak": peak,
                     "unit": "GB/s", "frac": round(conv_gbs / peak, 4),
                     "traffic": int(traffic * n / 256.0) if traffic else None,
                     "peak_source": which, "algorithmic_bytes_per_launch": int(conv_bytes),
                     "launch": "one pass = 22 kernel launches", "ms": round(conv_ms, 4),
                     "ms_source": conv_src},
        "tensor_TOPS_algorithmic": round(RESNET_FLOP_PER_IMG * n * (4 if flex else 3)
                                         / (conv_ms * 1e-3) / 1e12, 2),
        "parity": parity,
    }
    net.close()
    return line


# ---- the reference arm of the ResNet-20 workloads ------------------------------------------------
def resnet_cpu_reference(n, steps, warmup, max_seconds=None):
    """The reference CPU transformer on the same network and batch size (all host cores through
    numpy's BLAS); without the reference tree, the numpy restatement on a 32-image sample."""
    cores = os.cpu_count() or 1
    fe = reference_frontend()
    if fe is not None:
        rng, ngt = fe
        out, params = reference_resnet20(rng, n)
        cpu = ngt.make_transformer_factory("cpu")()
        comp = cpu.computation(out, *params)
        x = cifar_like(100, n)
        for _ in range(max(1, warmup)):
            comp(x)
        t0 = time.perf_counter()
        comp(x)
        one = time.perf_counter() - t0
        reps = steps if max_seconds is None else int(max(1, min(steps, max_seconds / max(one, 1e-3))))
        t0 = time.perf_counter()
        for _ in range(reps):
            comp(x)
        dt = (time.perf_counter() - t0) / reps
        cpu.close()
        return {"value": round(n / dt, 1), "unit": "img/s", "cores": cores, "kind": "reference",
                "sample": "%d passes of a %d-image batch through the reference's CPUTransformer "
                          "(numpy engine; MKL-DNN absent), BuildResnet-20 without batch norm, "
                          "numpy BLAS threads = all %d cores" % (reps, n, cores),
                "ms_per_step": round(dt * 1e3, 2), "batch": n}
    weights = resnet_weights(0)
    n = 32
    x = np.random.RandomState(100).standard_normal((3, 32, 32, n)).astype(np.float32)
    resnet20_numpy(x, weights)
    t0 = time.perf_counter()
    resnet20_numpy(x, weights)
    one = time.perf_counter() - t0
    reps = steps if max_seconds is None else int(max(1, min(steps, max_seconds / max(one, 1e-3))))
    t0 = time.perf_counter()
    for _ in range(reps):
        resnet20_numpy(x, weights)
    dt = (time.perf_counter() - t0) / reps
    return {"value": round(n / dt, 1), "unit": "img/s", "cores": cores, "kind": "port",
            "sample": "%d passes of a %d-image batch through the numpy restatement of the "
                      "network (oracle/conv_oracle.py; the reference tree is absent here; numpy "
                      "BLAS threads = all %d cores)" % (reps, n, cores),
            "ms_per_step": round(dt * 1e3, 2), "batch": n}


# ---- ResNet-20 data-parallel training step (global batch fixed, split over the GPUs) -----------
class ResnetTraining(object):
    """One momentum-SGD step of ResNet-20 as a computation.  With the reference tree: the
    reference's builder, cross_entropy_multi, autodiff and GradientDescentMomentum(0.1, 0.9)
    through the plug-in (which places the gradient exchange where the reference's passes would,
    from the gradients' reduce_func tags).  Without: this package's hand-differentiated graph."""

    def __init__(self, torch, local, flex, global_n, rank, world, comm, bucket_bytes, lr,
                 min_buckets=0):
        n = global_n // world
        fe = reference_frontend()
        kw = dict(device_id=local, flex=flex, comm=comm)
        if bucket_bytes:
            kw["bucket_bytes"] = bucket_bytes
        if min_buckets:
            kw["min_buckets"] = min_buckets
        r = np.random.RandomState(3)
        labels = r.randint(0, 10, global_n)
        lo, hi = rank * n, (rank + 1) * n
        if fe is not None:
            rng, ngt = fe
            out, params = reference_resnet20(rng, n, train=True, lr=lr)
            self.outer_t = ngt.make_transformer_factory("b200", **kw)()
            self.call = self.outer_t.computation(out, *params)
            self.t, self.comp = self.outer_t.impl, self.call.impl
            self.frontend = "reference BuildResnet-20 + cross_entropy_multi + autodiff + " \
                            "GradientDescentMomentum via the ngraph plug-in"
            vals = [cifar_like(7, global_n)[..., lo:hi], labels[lo:hi].astype(np.float32)]
        else:
            import ngraph_python_b200 as ng
            from ngraph_python_b200 import configs
            self.outer_t = ng.transformers.allocate_transformer("b200", **kw)
            outs, params, vals = configs.resnet_train_step(ng, global_n=global_n,
                                                           shard=(rank, world), hw=32, blocks=3,
                                                           lr=lr)
            self.call = self.outer_t.computation(outs[0], *params)
            self.t, self.comp = self.outer_t, self.call
            self.frontend = "this package's hand-differentiated ResNet-20 (reference tree absent)"
        self.host = []
        for v in vals:
            pinned = torch.empty(v.shape, dtype=torch.float32).pin_memory()
            pinned.numpy()[...] = v
            self.host.append(pinned.numpy())

    def close(self):
        self.outer_t.close()


def measure_training(args, rank, world, torch, dist, local, flex, steps, repeats, with_e2e=True):
    """Times one training step; returns the fields of a bench line (rank 0) or None."""
    from ngraph_python_b200.comm import NcclComm, TorchDistComm, SingleProcessComm
    gn = args.global_batch
    if gn % world or (gn // world) % 128:
        raise SystemExit("global batch must give every GPU a multiple of 128 images")
    n = gn // world
    if dist is None:
        comm = SingleProcessComm()
    elif args.comm == "torch":
        comm = TorchDistComm()
    else:
        comm = NcclComm.from_torch_distributed(local)     # the library's own b2_comm_* group
    job = ResnetTraining(torch, local, flex, gn, rank, world, comm, args.bucket_bytes, lr=args.lr,
                         min_buckets=args.min_buckets)
    t, comp, host = job.t, job.comp, job.host
    losses = [float(job.call(*host)) for _ in range(3)]
    graphed = False
    if not args.no_graph:
        comp.capture()          # one graph per step, the NCCL exchanges inside it (--comm torch:
                                # graphs between the exchanges)
        graphed = True
    timer = Timer(torch, dist)

    def step_resident():
        t._begin_call(comp)
        comp.executor()
        t._end_call(comp)

    launches0 = t.kernel_launches
    for _ in range(args.warmup):
        step_resident()
    launches_per_step = (t.kernel_launches - launches0) // max(args.warmup, 1)
    sampler = ClockSampler(local)
    timer.barrier()
    sampler.start()
    loop_ms = timer.loops(step_resident, steps, repeats)
    # (the step exchanges gradients: the replicas must agree on how often they run it)
    sampler.keep_loaded(step_resident, torch.cuda.synchronize, dist=dist, torch=torch)
    stream = timer.stream
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
    e2e_steps = max(1, min(steps, args.e2e_steps * 2))
    e2e_ms = timer.wall(lambda: job.call(*host), e2e_steps) if with_e2e else None
    last = float(job.call(*host))
    clocks = sampler.stop()
    alone_ms = nocomm_ms = 0.0
    exchanged = []
    if dist is not None and t._allreduce is not None:
        # How much of the exchange the step hides.  (1) what one step exchanges, (2) the same
        # collectives alone, back to back, (3) the step with the collectives left out; exposed
        # time = step - step without exchange.  Done last: (3) lets the replicas drift apart.
        ar, real = t._allreduce, t._allreduce.comm
        step_resident()
        torch.cuda.synchronize()
        exchanged = [int(c) for c in ar.last_sizes]       # elements of every collective of a step
        bufs = [torch.zeros(c, dtype=torch.float32, device="cuda") for c in exchanged]

        def collectives_alone():
            for b in bufs:
                real.all_reduce_async(b, "mean").wait()
        timer.loops(collectives_alone, 3, 1)
        alone_ms = statistics.median(timer.loops(collectives_alone, 20, 3)) / 20
        ar.comm = SingleProcessComm()
        if graphed:
            comp.capture()                                 # the same step list without exchanges
        timer.loops(step_resident, 3, 1)
        nocomm_ms = statistics.median(timer.loops(step_resident, steps, repeats)) / steps
        ar.comm = real
    buckets = len(t._allreduce.plan.buckets) if t._allreduce is not None else 0
    n_steps = len(comp.steps)
    frontend = job.frontend
    job.close()
    if rank != 0:
        return None
    ms_step = statistics.median(loop_ms) / steps
    conv_ms = sum(kinds[k][0] for k in ("conv", "conv_bprop", "conv_update") if k in kinds) / passes
    tpeak, which = tensor_peak()
    tpeak = tpeak * 2 if flex else tpeak / 2
    tops = 3 * RESNET_FLOP_PER_IMG * n * (4 if flex else 3) / (conv_ms * 1e-3) / 1e12
    out = {
        "metric": "ResNet-20 %s data-parallel training img/s" % ("flex16" if flex else "fp32"),
        "value": round(gn / (ms_step * 1e-3), 1), "unit": "img/s", "n_gpus": world,
        "steps": steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 4),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "flex16 (i16 mantissas, int8 hi/lo tensor-core products, i32 accumulation)"
                 if flex else "f32 (3xTF32 tensor-core products)",
        "data": "synthetic",
        "config": {"workload": "resnet20_train_%s" % ("flex16" if flex else "fp32"),
                   "global_batch": gn, "batch_per_gpu": n,
                   "image": [3, 32, 32], "layout": "C,H,W,N",
                   "optimizer": "momentum 0.9 + Kahan, lr %g" % args.lr,
                   "network": frontend,
                   "parallelism": "dp%d" % world, "allreduce_buckets": buckets,
                   "exchange": type(comm).__name__,
                   "bucket_bytes": t.bucket_bytes, "steps_per_pass": n_steps,
                   "cuda_graph": graphed,
                   "l2": "each step streams >126 MB of activations, gradients and operand planes"},
        "clocks": clocks,
        "repeats": spread(loop_ms, steps),
        "gpu_launches": launches_per_step * steps,
        "roofline": {"bound": "tensor", "kernel": "convolution fprop + bprop + update steps",
                     "achieved": round(tops, 2), "peak": round(tpeak, 1),
                     "unit": "TOPS (int8)" if flex else "TFLOP/s (tf32)",
                     "frac": round(tops / tpeak, 4), "traffic": None,
                     "peak_source": which + (" bf16 x 2 as int8 stand-in" if flex else
                                             " bf16 / 2 as tf32 stand-in"),
                     "ms": round(conv_ms, 4)},
        "step_time_ms_by_kind": {k: round(v[0] / passes, 4) for k, v in kinds.items()},
        "allreduce_algorithmic_bytes_per_gpu": int(2 * (world - 1) / world * TRAIN_PARAM_BYTES),
        "loss_first_steps": [round(v, 5) for v in losses], "loss_last": round(last, 5),
    }
    if e2e_ms is not None:
        out["e2e"] = {"value": round(gn / (e2e_ms / e2e_steps * 1e-3), 1), "unit": "img/s",
                      "h2d_bytes_per_step": int(sum(h.nbytes for h in host)),
                      "d2h_bytes_per_step": 4, "steps": e2e_steps,
                      "ms_per_step": round(e2e_ms / e2e_steps, 3)}
    if exchanged:
        exposed = max(0.0, ms_step - nocomm_ms)
        out["allreduce"] = {
            "collectives_per_step": len(exchanged), "bytes_per_step": int(4 * sum(exchanged)),
            "alone_ms": round(alone_ms, 4), "step_without_exchange_ms": round(nocomm_ms, 4),
            "exposed_ms": round(exposed, 4),
            "overlap_frac": round(min(1.0, max(0.0, 1.0 - exposed / alone_ms)), 3) if alone_ms > 0 else None}
    return out


def run_resnet_train(args, rank, world, torch, dist, local):
    flex = args.workload == "resnet20_train_flex16"
    line = measure_training(args, rank, world, torch, dist, local, flex, args.steps, args.repeats)
    if line is not None and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = train_cpu_reference(args.global_batch, steps=1, lr=args.lr)
    return line


def train_cpu_reference(global_n, steps=1, lr=0.1):
    """The reference CPU transformer on one training step of the global batch (hetr itself needs
    mpirun / MLSL, which this image lacks)."""
    cores = os.cpu_count() or 1
    fe = reference_frontend()
    if fe is not None:
        rng, ngt = fe
        out, params = reference_resnet20(rng, global_n, train=True, lr=lr)
        cpu = ngt.make_transformer_factory("cpu")()
        comp = cpu.computation(out, *params)
        vals = [cifar_like(7, global_n),
                np.random.RandomState(3).randint(0, 10, global_n).astype(np.float32)]
        comp(*vals)
        t0 = time.perf_counter()
        for _ in range(steps):
            comp(*vals)
        dt = (time.perf_counter() - t0) / steps
        cpu.close()
        return {"value": round(global_n / dt, 2), "unit": "img/s", "cores": cores,
                "kind": "reference",
                "sample": "%d training step(s) of the global batch of %d images on the "
                          "reference's CPUTransformer (numpy engine, numpy BLAS threads = all %d "
                          "cores)" % (steps, global_n, cores),
                "ms_per_step": round(dt * 1e3, 1)}
    import ngraph_python_b200 as ng
    from ngraph_python_b200 import configs
    from tests import mirror_interp
    gn = 32
    outs, params, vals = configs.resnet_train_step(ng, global_n=gn, hw=32, blocks=3, lr=lr)
    interp = mirror_interp.Interp()
    t0 = time.perf_counter()
    for _ in range(steps):
        interp.run(outs[:1], dict(zip(params, vals)))
    dt = (time.perf_counter() - t0) / steps
    return {"value": round(gn / dt, 2), "unit": "img/s", "cores": cores, "kind": "port",
            "sample": "%d training step(s) on a %d-image batch, numpy restatement of every op "
                      "(reference tree absent; numpy BLAS threads = all %d cores)"
                      % (steps, gn, cores),
            "ms_per_step": round(dt * 1e3, 1)}


# ---- configuration 3: GEMM --------------------------------------------------------------------
def int8_yardstick(torch, n=8192, reps=10):
    """A library int8 GEMM (torch._int_mm -> cuBLASLt), used ONLY as the measured denominator of
    the flex16 GEMM's roofline fraction: best of `reps`, TOPS (2 n^3 / t)."""
    try:
        a = torch.randint(-127, 128, (n, n), dtype=torch.int8, device="cuda")
        b = torch.randint(-127, 128, (n, n), dtype=torch.int8, device="cuda")
        for _ in range(3):
            torch._int_mm(a, b)
        best = None
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._int_mm(a, b)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            best = ms if best is None else min(best, ms)
        del a, b
        return 2.0 * n ** 3 / (best * 1e-3) / 1e12
    except Exception:       # pragma: no cover  (yardstick only: absence changes no result)
        return None


def measure_gemm(args, rank, world, torch, dist, local, flex, size, steps, repeats,
                 with_e2e=True):
    import ngraph_python_b200 as ng
    n = size
    t = ng.transformers.allocate_transformer("b200", device_id=local, flex=flex)
    M, K, N = ng.make_axis(n, name="M"), ng.make_axis(n, name="K"), ng.make_axis(n, name="N")
    a, b = ng.placeholder([M, K]), ng.placeholder([K, N])
    c = ng.dot(a, b)
    cvar = ng.persistent_tensor([M, N])
    # C stays on the device (assigned to a persistent tensor); its column maxima are returned
    out = ng.sequential([ng.assign(cvar, c), ng.max(cvar, reduction_axes=[M])])
    comp = t.computation(out, a, b)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(rank)
    dev = []
    for scale in ((2.0 ** -15, 2.0 ** -12) if flex else (1.0, 1.0)):
        if flex:
            v = torch.randint(-32767, 32768, (n, n), device="cuda", generator=gen).float() * scale
        else:
            v = torch.randn((n, n), device="cuda", generator=gen)
        dev.append(v)
    comp(*dev)
    comp(*dev)
    gemm_step = [s for s in comp.steps if s.kind == "gemm"][0]
    timer = Timer(torch, dist)
    for _ in range(args.warmup):
        t._launch_step(gemm_step)
    sampler = ClockSampler(local)
    timer.barrier()
    sampler.start()
    loop_ms = timer.loops(lambda: t._launch_step(gemm_step), steps, repeats)
    sampler.keep_loaded(lambda: t._launch_step(gemm_step), torch.cuda.synchronize)
    e2e = None
    if with_e2e:
        host = []
        for v in dev:
            pinned = torch.empty((n, n), dtype=torch.float32).pin_memory()
            pinned.copy_(v)
            host.append(pinned.numpy())
        comp(*host)
        e2e_steps = max(1, min(steps, args.e2e_steps))
        e2e_ms = timer.wall(lambda: comp(*host), e2e_steps)
        e2e = (e2e_ms, e2e_steps, int(sum(h.nbytes for h in host)))
    clocks = sampler.stop()
    launches = gemm_step.launches
    del dev
    t.close()
    yard = int8_yardstick(torch) if (flex and rank == 0) else None
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    ms_step = statistics.median(loop_ms) / steps
    ops = 2.0 * n * n * n
    bf16, which = tensor_peak()
    # flex16: four int8 products per MAC
    tensor_ops = (4 if flex else 3) * ops
    achieved = tensor_ops / (ms_step * 1e-3) / 1e12
    if flex and yard:
        peak, src = yard, "library int8 GEMM (torch._int_mm, %d^3, best of 10) measured in this run" % 8192
    elif flex:
        peak, src = 2 * bf16, which + " bf16 x2 as int8 stand-in"
    else:
        peak, src = bf16 / 2, which + " bf16 / 2 as tf32 stand-in"
    line = {
        "metric": "%s GEMM T%sMAC-op/s (2MNK/t), M=N=K=%d" % ("flex16" if flex else "fp32",
                                                              "flex-" if flex else "", n),
        "value": round(world * ops / (ms_step * 1e-3) / 1e12, 2), "unit": "Tops/s",
        "n_gpus": world, "steps": steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None,
        "dtype": "flex16 (int8 hi/lo tensor-core products, i32 accumulation)" if flex
                 else "f32 (3xTF32)",
        "data": "synthetic",
        "config": {"workload": "gemm_%s" % ("flex16" if flex else "fp32"), "M": n, "N": n, "K": n,
                   "replicas": world,
                   "l2": "operand planes (%d MB) larger than L2" % (4 * n * n * (1 if flex else 4) >> 20)
                         if n >= 8192 else "operands fit in L2 at this size",
                   "includes": "operand split pre-pass + tensor-core kernel"},
        "clocks": clocks,
        "repeats": spread(loop_ms, steps),
        "gpu_launches": launches * steps,
        "roofline": {"bound": "tensor", "achieved": round(achieved, 1), "peak": round(peak, 1),
                     "unit": "TOPS (int8)" if flex else "TFLOP/s (tf32)",
                     "frac": round(achieved / peak, 4), "traffic": None,
                     "peak_source": src, "algorithmic_ops_per_launch": tensor_ops},
    }
    if flex:
        line["roofline"]["frac_of_datasheet_4500_TOPS"] = round(achieved / INT8_DATASHEET_TOPS, 4)
        line["roofline"]["frac_of_2x_measured_bf16"] = round(achieved / (2 * bf16), 4)
    if e2e is not None:
        e2e_ms, e2e_steps, nbytes = e2e
        line["e2e"] = {"value": round(world * ops / (e2e_ms / e2e_steps * 1e-3) / 1e12, 3),
                       "unit": "Tops/s", "h2d_bytes_per_step": nbytes,
                       "d2h_bytes_per_step": int(n * (2 if flex else 4)), "steps": e2e_steps,
                       "ms_per_step": round(e2e_ms / e2e_steps, 3)}
    return line


# ---- configuration 2: fused elementwise + reductions --------------------------------------------
def build_c2(ng, rows, cols):
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


def measure_c2(args, rank, world, torch, dist, local, flex, rows, steps, repeats, with_e2e=True):
    import ngraph_python_b200 as ng
    cols = C2_COLS
    t = ng.transformers.allocate_transformer("b200", device_id=local, flex=flex)
    outs, params = build_c2(ng, rows, cols)
    comp = t.computation(outs, *params)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(rank)
    dev = [torch.randn((rows, cols), device="cuda", generator=gen) for _ in range(4)]
    comp(*dev)            # compile, first-call exponent initialisation
    res = comp(*dev)
    timer = Timer(torch, dist)
    launches0 = t.kernel_launches
    for _ in range(args.warmup):
        comp.executor()
    launches_per_step = (t.kernel_launches - launches0) // max(args.warmup, 1)
    sampler = ClockSampler(local)
    timer.barrier()
    sampler.start()
    loop_ms = timer.loops(comp.executor, steps, repeats)
    sampler.keep_loaded(comp.executor, torch.cuda.synchronize)
    e2e = None
    if with_e2e:
        host = []
        for v in dev:
            pinned = torch.empty((rows, cols), dtype=torch.float32).pin_memory()
            pinned.copy_(v)
            host.append(pinned.numpy())
        comp(*host)
        e2e_steps = max(1, min(steps, args.e2e_steps))
        e2e_ms = timer.wall(lambda: comp(*host), e2e_steps)
        e2e = (e2e_ms, e2e_steps, int(sum(h.nbytes for h in host)))
    clocks = sampler.stop()
    d2h = sum(np.asarray(r).size for r in res) * (2 if flex else 4)
    del dev
    t.close()
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    alg = c2_algorithmic_bytes(flex, rows, cols)
    ms_step = statistics.median(loop_ms) / steps
    gbs = world * alg / (ms_step * 1e-3) / 1e9
    peak, which = peaks()
    kernel_gbs = alg / (ms_step * 1e-3) / 1e9
    name = "c2_flex16" if flex else "c2_fp32"
    traffic = NCU_TRAFFIC_BYTES.get(name)
    line = {
        "metric": "fused-EW HBM GB/s (y=tanh(a*x+b)*sigmoid(c), row sum and row maxabs)",
        "value": round(gbs, 1), "unit": "GB/s", "n_gpus": world, "steps": steps,
        "warmup": args.warmup, "ms_per_step": round(ms_step, 5), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None,
        "dtype": "flex16 (i16 mantissa storage, f32 math)" if flex else "f32",
        "data": "synthetic",
        "config": {"workload": name, "shape": [rows, cols], "replicas": world,
                   "l2": "inputs (%d MB) larger than L2" % (4 * rows * cols * (2 if flex else 4) >> 20),
                   "fused_ops": 11, "y_materialised": True},
        "clocks": clocks,
        "repeats": spread(loop_ms, steps),
        "gpu_launches": launches_per_step * steps,
        "roofline": {"bound": "hbm", "achieved": round(kernel_gbs, 1), "peak": peak,
                     "unit": "GB/s", "frac": round(kernel_gbs / peak, 4),
                     "traffic": int(traffic * rows / C2_ROWS) if traffic else None,
                     "peak_source": which, "algorithmic_bytes_per_launch": alg},
    }
    if e2e is not None:
        e2e_ms, e2e_steps, nbytes = e2e
        line["e2e"] = {"value": round(world * alg / (e2e_ms / e2e_steps * 1e-3) / 1e9, 2),
                       "unit": "GB/s", "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": d2h,
                       "steps": e2e_steps, "ms_per_step": round(e2e_ms / e2e_steps, 3)}
    return line


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


def c2_cpu_reference(workload, rows, steps, warmup):
    """(GB/s, seconds per pass, cores, kind, what) for `rows` rows of configuration 2 on the host:
    the reference CPU transformer on the same graph (fp32); flex16 has no CPU implementation in the
    reference (its flex transformer is GPU-only), so the numpy restatement under oracle/ is timed."""
    flex = workload == "c2_flex16"
    cores = os.cpu_count() or 1
    rng_ = np.random.RandomState(0)
    vals = [rng_.standard_normal((rows, C2_COLS)).astype(np.float32) for _ in range(4)]
    fe = reference_frontend()
    if fe is not None and not flex:
        rng, ngt = fe
        outs, params = build_c2(rng, rows, C2_COLS)
        cpu = ngt.make_transformer_factory("cpu")()
        comp = cpu.computation(outs, *params)

        def one():
            comp(*vals)
        kind = "reference"
        what = "reference CPUTransformer on the same graph (one numpy pass per op)"
    else:
        from concurrent.futures import ThreadPoolExecutor
        blocks = np.array_split(np.arange(rows), min(cores, rows))

        def one():
            with ThreadPoolExecutor(cores) as ex:
                list(ex.map(lambda idx: _c2_cpu_block(flex, [v[idx] for v in vals]), blocks))
        kind = "port"
        what = "numpy restatement (oracle/), row blocks on %d threads" % cores
    for _ in range(max(1, warmup)):
        one()
    t0 = time.perf_counter()
    for _ in range(steps):
        one()
    dt = (time.perf_counter() - t0) / steps
    alg = c2_algorithmic_bytes(flex, rows, C2_COLS)
    return alg / dt / 1e9, dt, cores, kind, what


def c2_cpu_baseline(workload, max_seconds=10.0):
    rows = 256
    gbs, dt, cores, kind, what = c2_cpu_reference(workload, rows, steps=1, warmup=1)
    steps = int(max(1, min(20, max_seconds / max(dt, 1e-3))))
    gbs, dt, cores, kind, what = c2_cpu_reference(workload, rows, steps=steps, warmup=0)
    return {"value": round(gbs, 3), "unit": "GB/s", "cores": cores, "kind": kind,
            "sample": "%d of %d rows x %d cols, %d passes, %s" % (rows, C2_ROWS, C2_COLS, steps, what)}


# ---------------------------------------------------------------------------------------------
def slim(line, keys=("metric", "value", "unit", "ms_per_step", "config", "roofline", "repeats",
                     "gpu_launches", "allreduce", "step_time_ms_by_kind", "loss_first_steps",
                     "loss_last", "clocks", "scaling")):
    return {k: line[k] for k in keys if k in line} if line else None


def run_b200(args, rank, world):
    import torch
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        # (a replica that fails must not keep the others in a collective for the default 10 min)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local),
                                timeout=datetime.timedelta(seconds=240))
    try:
        w = args.workload
        if w.startswith("gemm"):
            return measure_gemm(args, rank, world, torch, dist, local, w == "gemm_flex16",
                                args.size, args.steps, args.repeats)
        if w.startswith("resnet20_train"):
            return run_resnet_train(args, rank, world, torch, dist, local)
        if w.startswith("c2"):
            line = measure_c2(args, rank, world, torch, dist, local, w == "c2_flex16", args.rows,
                              args.steps, args.repeats)
            if line is not None and world == 1 and not args.no_cpu_baseline:
                line["cpu_baseline"] = c2_cpu_baseline(w)
            return line
        line = run_resnet(args, rank, world, torch, dist, local)
        torch.cuda.empty_cache()
        if w == "resnet20_flex16" and not args.no_extras and args.batch == RESNET_N:
            # the rest of the headline metric, in the same driver-run line
            extras = {}
            if world == 1:
                extras["c2_flex16"] = slim(measure_c2(args, rank, world, torch, dist, local, True,
                                                      C2_ROWS, 20, 3, with_e2e=False))
                extras["c2_fp32"] = slim(measure_c2(args, rank, world, torch, dist, local, False,
                                                    C2_ROWS, 20, 3, with_e2e=False))
                extras["gemm_flex16_8192"] = slim(measure_gemm(args, rank, world, torch, dist,
                                                               local, True, 8192, 10, 3,
                                                               with_e2e=False))
            extras["resnet20_train_flex16"] = slim(measure_training(
                args, rank, world, torch, dist, local, True, 10, 3, with_e2e=False))
            if line is not None:
                line["extras"] = extras
        if line is not None and world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = resnet_cpu_reference(args.batch, steps=10, warmup=1,
                                                        max_seconds=12.0)
        return line
    finally:
        if dist is not None:
            dist.destroy_process_group()


def run_reference(args, rank, world):
    """The reference's CPU implementation of the workload on the host cores (rank 0 only)."""
    if rank != 0:
        return None
    cores = os.cpu_count() or 1
    w = args.workload
    zero_copy = {"h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    if w.startswith("gemm"):
        n = min(args.size, 2048)
        flex = w == "gemm_flex16"
        r = np.random.RandomState(0)
        fe = reference_frontend()
        av = r.randint(-32767, 32768, (n, n)).astype(np.float32)
        bv = r.randint(-32767, 32768, (n, n)).astype(np.float32)
        if fe is not None:
            rng, ngt = fe
            M, K, N = [rng.make_axis(n, name=nm) for nm in ("M", "K", "N")]
            a, b = rng.placeholder([M, K]), rng.placeholder([K, N])
            cpu = ngt.make_transformer_factory("cpu")()
            comp = cpu.computation(rng.dot(a, b), a, b)
            one, kind = (lambda: comp(av, bv)), "reference"
            what = "reference CPUTransformer DotOp (np.dot, cpu/cpuengine.py:339-350)"
        else:
            one, kind, what = (lambda: av @ bv), "port", "numpy matmul"
        one()
        t0 = time.perf_counter()
        for _ in range(max(1, args.steps)):
            one()
        dt = (time.perf_counter() - t0) / max(1, args.steps)
        v = round(2.0 * n ** 3 / dt / 1e12, 4)
        base = {"value": v, "unit": "Tops/s", "cores": cores, "kind": kind,
                "sample": "%s, %d^3 (bounded from %d^3), %d BLAS threads" % (what, n, args.size, cores)}
        return {"impl": "reference", "metric": "%s GEMM T%sMAC-op/s (2MNK/t), M=N=K=%d"
                % ("flex16" if flex else "fp32", "flex-" if flex else "", args.size), "value": v,
                "unit": "Tops/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f32 (numpy)", "data": "synthetic",
                "config": {"workload": w, "M": args.size, "N": args.size, "K": args.size},
                "cpu_baseline": base, "e2e": dict(value=v, unit="Tops/s", **zero_copy),
                "gpu_launches": 0}
    if w.startswith("resnet20_train"):
        flex = w == "resnet20_train_flex16"
        b = train_cpu_reference(args.global_batch, steps=max(1, min(args.steps, 3)), lr=args.lr)
        return {
            "impl": "reference",
            "metric": "ResNet-20 %s data-parallel training img/s" % ("flex16" if flex else "fp32"),
            "value": b["value"], "unit": "img/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": b["ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32 (numpy)", "data": "synthetic",
            "config": {"workload": w, "global_batch": args.global_batch,
                       "image": [3, 32, 32], "layout": "C,H,W,N"},
            "cpu_baseline": b, "e2e": dict(value=b["value"], unit="img/s", **zero_copy),
            "gpu_launches": 0,
        }
    if w.startswith("resnet20"):
        flex = w == "resnet20_flex16"
        b = resnet_cpu_reference(args.batch, steps=max(1, args.steps), warmup=max(1, args.warmup),
                                 max_seconds=120.0)
        fe = reference_frontend()
        frontend = REFERENCE_NETWORK if fe is not None else OWN_NETWORK
        return {
            "impl": "reference",
            "metric": "ResNet-20 %s inference img/s" % ("flex16" if flex else "fp32"),
            "value": b["value"], "unit": "img/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": b["ms_per_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32 (numpy)", "data": "synthetic",
            "config": resnet_config(w, b["batch"], world, frontend),
            "cpu_baseline": b, "e2e": dict(value=b["value"], unit="img/s", **zero_copy),
            "gpu_launches": 0,
        }
    rows = 256
    gbs, dt, cores, kind, what = c2_cpu_reference(w, rows, max(1, args.steps), max(0, args.warmup))
    flex = w == "c2_flex16"
    return {
        "impl": "reference",
        "metric": "fused-EW HBM GB/s (y=tanh(a*x+b)*sigmoid(c), row sum and row maxabs)",
        "value": round(gbs, 3), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None,
        "dtype": "flex16 (i16 mantissa storage, f32 math)" if flex else "f32",
        "data": "synthetic",
        "config": {"workload": w, "shape": [C2_ROWS, C2_COLS], "replicas": world},
        "cpu_baseline": {"value": round(gbs, 3), "unit": "GB/s", "cores": cores, "kind": kind,
                         "sample": "each step = %d of %d rows x %d cols, %s"
                                   % (rows, C2_ROWS, C2_COLS, what)},
        "e2e": dict(value=round(gbs, 3), unit="GB/s", **zero_copy),
        "gpu_launches": 0,
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--repeats", type=int, default=5,
                    help="the timed loop of --steps steps is run this many times; median reported")
    ap.add_argument("--workload", default="resnet20_flex16",
                    choices=["resnet20_flex16", "resnet20_fp32", "c2_flex16", "c2_fp32",
                             "gemm_flex16", "gemm_fp32", "resnet20_train_flex16",
                             "resnet20_train_fp32"])
    ap.add_argument("--global-batch", type=int, default=1024,
                    help="images per training step over all GPUs (training workloads)")
    ap.add_argument("--bucket-bytes", type=int, default=0,
                    help="upper bound of an allreduce bucket (0: the library's default)")
    ap.add_argument("--min-buckets", type=int, default=0,
                    help="lower bound on the buckets of a step (0: the library's default, 4)")
    ap.add_argument("--size", type=int, default=8192, help="M = N = K of the GEMM workloads")
    ap.add_argument("--batch", type=int, default=RESNET_N, help="images per GPU (ResNet-20)")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--rows", type=int, default=C2_ROWS,
                    help="rows of the microbenchmark (smaller values are for profiler captures)")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="default workload only: leave out configurations 2, 3 and 5")
    ap.add_argument("--lr", type=float, default=0.1, help="learning rate (training workloads)")
    ap.add_argument("--comm", default="b2", choices=["b2", "torch"],
                    help="gradient exchange through the library's NCCL group or torch.distributed")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch kernel by kernel instead of replaying a CUDA graph")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    # whatever the libraries print on the way (NCCL writes its version to file descriptor 1) goes
    # to stderr: stdout carries the one JSON line
    sys.stdout.flush()
    real_fd = os.dup(1)
    os.dup2(2, 1)
    out, sys.stdout = sys.stdout, sys.stderr
    try:
        if args.impl == "reference":
            line = run_reference(args, rank, world)
        else:
            line = run_b200(args, rank, world)
    finally:
        sys.stdout = out
        os.dup2(real_fd, 1)
        os.close(real_fd)
    if line is not None:
        print(json.dumps(line))
        sys.stdout.flush()


if __name__ == "__main__":
    main()
