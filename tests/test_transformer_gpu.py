"""GPU parity of the b200 transformer, through transformer.computation(), against fixtures made
by the reference's own CPU transformer (tests/golden/make_fixtures.py) on the same seeded inputs.

fp32 bar: rtol 1e-4 / atol 1e-5 (sums scaled by the number of terms).
flex16 bar: the reference's flex tolerance, rtol 1e-2 / atol 8 * 2**-dec(max|expected|)
(ngraph/transformers/flexgputransform.py:80-103)."""
import os

import numpy as np
import pytest

import ngraph_python_b200 as ng
from tests.flexsim import flex_tolerance
from tests.golden import cases

pytestmark = pytest.mark.gpu
FIX = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "fixtures")


def _run(name, **kw):
    outs, params, vals = cases.CASES[name](ng)
    t = ng.transformers.allocate_transformer("b200", **kw)
    comp = t.computation(outs, *params)
    results = []
    for rep in range(cases.REPEAT.get(name, 1)):
        results.append([np.array(r, copy=True) for r in comp(*vals)])
    launches = comp.launches_per_call
    t.close()
    return results, launches


def _n_terms(name, k, expected, outs_shape0):
    return 1


@pytest.mark.parametrize("fuse", [True, False])
@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_fp32_matches_reference_cpu(name, fuse):
    fix = np.load(os.path.join(FIX, name + ".npz"))
    results, launches = _run(name, fuse=fuse)
    for rep, res in enumerate(results):
        for k, got in enumerate(res):
            exp = fix["out%d_%d" % (rep, k)]
            assert got.shape == exp.shape, (name, k)
            # a sum of n terms carries n roundings: scale atol with the magnitude of the result
            atol = 1e-5 * max(1.0, float(np.max(np.abs(exp))))
            np.testing.assert_allclose(got, exp, rtol=1e-4, atol=atol,
                                       err_msg="%s output %d call %d" % (name, k, rep))


def test_fusion_reduces_launches():
    _, fused = _run("c2_fused", fuse=True)
    _, unfused = _run("c2_fused", fuse=False)
    assert fused == 1
    assert unfused >= 10     # the reference's one-kernel-per-op count for this graph


# (batchnorm_train is fp32 only: the reference's flex transformer does not run batch normalisation
# either -- ngraph/frontends/neon/tests/test_batchnorm_layer.py:148,251 skip it -- and the running
# statistics, which start at 0 and 1 and grow by a tenth of the batch value per call, overrun
# the exponent autoflex picks from their history)
FLEX_CASES = ["c2_fused", "ew_4d", "reduce_4d_axis1", "recip_add_sum", "broadcast_bias",
              "assign_sequence", "conv_basic", "conv_stride2_1x1", "conv_stride2_3x3", "conv_grads",
              "conv_grads_stride2", "mlp_forward", "pool_max", "pool_grads", "pool_grads_avg",
              "lut_embedding", "lut_embedding_axis1",
              "resnet8_small", "resnet20"]


@pytest.mark.parametrize("fuse", [True, False])
@pytest.mark.parametrize("name", FLEX_CASES)
def test_flex16_within_reference_tolerance(name, fuse):
    fix = np.load(os.path.join(FIX, name + ".npz"))
    results, _ = _run(name, flex=True, fuse=fuse)
    for rep, res in enumerate(results):
        for k, got in enumerate(res):
            exp = fix["out%d_%d" % (rep, k)]
            atol, rtol = flex_tolerance(exp)
            # the fixture is the fp32 result: the flex inputs' own quantisation error (and, with
            # one kernel per op, that of every intermediate) propagates through the products
            atol *= 4
            np.testing.assert_allclose(got, exp, rtol=rtol, atol=atol,
                                       err_msg="%s output %d call %d" % (name, k, rep))


@pytest.mark.parametrize("flex", [False, True])
def test_captured_graph_matches_stepwise(flex):
    """Two transformers see the same sequence of calls; one of them switches to replaying a
    captured CUDA graph half way.  Results must be identical call by call -- also in flex mode,
    where exponents move between calls and the replay has to pick them up from the device table."""
    def run(capture_after):
        outs, params, vals = cases.CASES["resnet8_small"](ng)
        seq = [vals, [v * 1.7 for v in vals], [v * 1.7 for v in vals], vals, [v * 0.3 for v in vals]]
        t = ng.transformers.allocate_transformer("b200", flex=flex)
        comp = t.computation(outs, *params)
        got = []
        for i, v in enumerate(seq):
            if i == capture_after:
                comp.capture()
            got.append([np.array(r, copy=True) for r in comp(*v)])
        t.close()
        return got
    stepwise, replayed = run(None), run(2)
    for a, b in zip(stepwise, replayed):
        for x, y in zip(a, b):
            assert np.array_equal(x, y)


def test_reduction_reads_assignment_from_registers():
    A, B = ng.make_axis(70, name="A"), ng.make_axis(33, name="B")
    x = ng.placeholder([A, B])
    keep = ng.persistent_tensor([A, B])
    out = ng.sequential([ng.assign(keep, x * 2.0), ng.max(keep, reduction_axes=[A])])
    t = ng.transformers.allocate_transformer("b200")
    comp = t.computation([out, keep], x)
    xv = np.random.RandomState(4).standard_normal((70, 33)).astype(np.float32)
    got, kept = comp(xv)
    np.testing.assert_allclose(got, (2 * xv).max(axis=0), rtol=1e-6)
    np.testing.assert_allclose(kept, 2 * xv, rtol=1e-6)
    t.close()


def test_conv_tails_fused_into_the_convolution_step():
    """Batch 128 takes the implicit-GEMM kernel, where `+ bias`, `+ residual` and ReLU after a
    convolution run in its epilogue (one launch per layer).  The result must agree with the
    unfused plan and with the numpy evaluation of the same graph, at flex16 tolerance."""
    from tests.mirror_interp import Interp
    res = {}
    for tail in (True, False):
        outs, params, vals = cases.resnet20(ng, n=128, hw=16, blocks=1)
        t = ng.transformers.allocate_transformer("b200", flex=True, fuse_conv_tail=tail)
        comp = t.computation(outs, *params)
        res[tail] = [[np.array(r, copy=True) for r in comp(*vals)] for _ in range(2)]
        kinds = [s.kind for s in comp.steps]
        if tail:
            assert kinds.count("ew") <= 4 and kinds.count("conv") == 10
            assert all(getattr(s, "epi", None) for s in comp.steps if s.kind == "conv")
        else:
            assert kinds.count("ew") >= 10
        t.close()
    outs, params, vals = cases.resnet20(ng, n=128, hw=16, blocks=1)
    exp = Interp().run(outs, dict(zip(params, vals)))
    for rep in range(2):
        for k in range(2):
            atol, rtol = flex_tolerance(exp[k])
            np.testing.assert_allclose(res[True][rep][k], exp[k], rtol=rtol, atol=4 * atol)
            np.testing.assert_allclose(res[True][rep][k], res[False][rep][k], rtol=rtol, atol=4 * atol)


def test_cached_filter_planes_follow_the_filters():
    """The convolution step keeps the byte planes of its filters until the filters change.  Another
    computation of the same transformer overwrites the filters; the next call -- step by step and
    as a replayed CUDA graph -- must see the new ones."""
    from oracle import conv_oracle as co
    Cc, K, H, W, N = 16, 16, 6, 6, 128
    ax = lambda n, nm: ng.make_axis(n, name=nm)   # noqa: E731
    ax_i = [ax(Cc, "C"), ax(1, "D"), ax(H, "H"), ax(W, "W"), ax(N, "N")]
    ax_f = [ax_i[0], ax(1, "T"), ax(3, "R"), ax(3, "S"), ax(K, "K")]
    ax_o = [ax_f[4], ax(1, "M"), ax(H, "P"), ax(W, "Q"), ax_i[4]]
    rng = np.random.RandomState(9)
    f0 = (rng.standard_normal((Cc, 1, 3, 3, K)) * 0.2).astype(np.float32)
    f1 = (rng.standard_normal((Cc, 1, 3, 3, K)) * 0.2).astype(np.float32)
    xv = rng.standard_normal((Cc, 1, H, W, N)).astype(np.float32)
    params = dict(pad_d=0, pad_h=1, pad_w=1, str_d=1, str_h=1, str_w=1, dil_d=1, dil_h=1, dil_w=1)
    for graph in (False, True):
        t = ng.transformers.allocate_transformer("b200", flex=True)
        x = ng.placeholder(ax_i)
        filt = ng.variable(ax_f, initial_value=f0)
        newf = ng.placeholder(ax_f)
        conv = t.computation(ng.convolution(params, x, filt, axes=ax_o), x)
        setf = t.computation(ng.assign(filt, newf), newf)
        a = np.array(conv(xv), copy=True)
        conv(xv)
        if graph:
            conv.capture()
            conv(xv)
        setf(f1)
        b = np.array(conv(xv), copy=True)
        for got, f in ((a, f0), (b, f1)):
            exp = co.conv_fprop(xv[:, 0], f[:, 0], (1, 1), (1, 1))
            tol = float(np.abs(exp).max()) * 2.0 ** -12
            assert np.abs(got[:, 0] - exp).max() <= 4 * tol
        assert np.abs(a - b).max() > 0.1
        t.close()


@pytest.mark.gpu
@pytest.mark.parametrize("case", ["assign_sequence", "mlp_train_step", "resnet_train_step"])
def test_flex_register_forwarding_is_bit_exact(case):
    """flex16: a kernel that goes on computing with a tensor it has just assigned reads the
    register through a requant op -- the mantissa the store writes times the tensor's step -- so
    the results are, bit for bit, those of separate kernels that reload the stored tensor."""
    got = {}
    for fw in (True, False):
        outs, params, vals = cases.CASES[case](ng)
        t = ng.transformers.allocate_transformer("b200", flex=True, forward_inplace=fw)
        comp = t.computation(outs, *params)
        got[fw] = [[np.array(r, copy=True) for r in comp(*vals)] for _ in range(3)]
        got[fw].append(len(comp.steps))
        t.close()
    assert got[True][-1] <= got[False][-1]
    if case != "mlp_train_step":                   # (plain SGD never reads a weight back)
        assert got[True][-1] < got[False][-1]      # fewer kernels
    for a, b in zip(got[True][:-1], got[False][:-1]):
        for x, y in zip(a, b):
            assert np.array_equal(x, y)


@pytest.mark.parametrize("flex", [False, True])
def test_device_tensor_get_slice_and_assign(flex):
    """Tensors read and written from the host outside any computation: whole tensor, windows
    (slices, integers, Ellipsis, steps), scalar fills -- GPUDeviceTensor.get / __getitem__ /
    __setitem__ of the reference (ngraph/transformers/gputransform.py:679-909); flex16 values go
    through value / scale, clip, truncate (flexgputransform.py:183-208)."""
    A, B, C = ng.make_axis(12, name="A"), ng.make_axis(9, name="B"), ng.make_axis(20, name="C")
    rng = np.random.RandomState(5)
    w0 = rng.uniform(-2, 2, (12, 9, 20)).astype(np.float32)
    w = ng.variable([A, B, C], initial_value=w0)
    x = ng.placeholder([A, B, C])
    t = ng.transformers.allocate_transformer("b200", flex=flex)
    comp = t.computation(w + x, x)
    t.initialize()
    dt = t.device_tensor(w)
    assert dt.shape == (12, 9, 20)
    step = dt.scale if flex else 0.0
    ref = w0.copy()
    if flex:
        ref = np.trunc(ref / step) * step          # the host write truncates
    np.testing.assert_allclose(dt.get(), ref, rtol=0, atol=1e-7)
    np.testing.assert_allclose(dt[2:5, :, 3].get(), ref[2:5, :, 3], rtol=0, atol=1e-7)
    np.testing.assert_allclose(dt[..., 1:20:3].get(), ref[..., 1:20:3], rtol=0, atol=1e-7)
    np.testing.assert_allclose(dt[-1].get(), ref[-1], rtol=0, atol=1e-7)
    new = rng.uniform(-1, 1, (3, 9)).astype(np.float32)
    dt[2:5, :, 3] = new
    dt[0, 1:4] = 0.5
    ref[2:5, :, 3] = np.trunc(new / step) * step if flex else new
    ref[0, 1:4] = 0.5
    np.testing.assert_allclose(t.get_tensor_view_value(w), ref, rtol=0, atol=1e-7)
    # and the computation sees what was written
    xv = np.zeros((12, 9, 20), np.float32)
    np.testing.assert_allclose(comp(xv), ref, rtol=0, atol=2 * step + 1e-7)
    dt[...] = w0 * 0.5
    got = dt.get()
    np.testing.assert_allclose(got, w0 * 0.5, rtol=0, atol=step + 1e-7)
    with pytest.raises(IndexError):
        dt[0, 0, 0, 0]
    with pytest.raises(ValueError):
        dt[2:5, :, 3] = np.zeros((9, 3), np.float32)
    t.close()


def test_tracing_writes_a_chrome_trace(tmp_path, monkeypatch):
    """TRACING=1 (the reference's switch, ngraph/util/trace_events.py:21-23): every step of every
    call becomes an 'X' event with a device timestamp and duration, written as Chrome-trace JSON
    when the transformer closes; results are those of an untraced run."""
    import json
    outs, params, vals = cases.CASES["resnet8_small"](ng)
    plain = ng.transformers.allocate_transformer("b200")
    want = [np.array(r, copy=True) for r in plain.computation(outs, *params)(*vals)]
    plain.close()
    monkeypatch.setenv("TRACING", "1")
    name = str(tmp_path / "trace")
    outs, params, vals = cases.CASES["resnet8_small"](ng)
    t = ng.transformers.allocate_transformer("b200", trace_name=name)
    comp = t.computation(outs, *params)
    for _ in range(2):
        got = comp(*vals)
    n_steps = len(comp.steps)
    t.close()
    for g_, w_ in zip(got, want):
        assert np.array_equal(g_, w_)
    trace = json.load(open(name + ".json"))["traceEvents"]
    assert len(trace) == 2 * n_steps
    assert all(e["ph"] == "X" and e["dur"] > 0 and e["ts"] >= 0 for e in trace)
    assert {e["cat"] for e in trace} >= {"conv", "ew", "gemm"}
    ts = [e["ts"] for e in trace]
    assert ts == sorted(ts)
