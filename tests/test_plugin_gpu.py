"""The b200 transformer EXECUTING behind the reference's own API on a GPU.

Graphs are built with the real `ngraph` package (the checker's copy under oracle/_ref, see
oracle/make_ref.py), compiled by `ngraph.transformers.make_transformer_factory('b200')()` --
the registration of ngraph/transformers/base.py:265-279, the computation protocol of
base.py:94-136, 420-433 -- and run on the device; the same graph runs through the reference's
CPU transformer ('cpu') on this machine's host cores and the two are compared.

fp32 bar: rtol 1e-4 / atol 1e-5 (atol scaled by the magnitude of a result that is a long sum).
flex16 bar: the reference's flex tolerance, rtol 1e-2 / atol 8 * 2**-dec(max|expected|)
(ngraph/transformers/flexgputransform.py:80-103), times 4 because the expectation is the fp32
result of the same graph, not a flex evaluation of it.
"""
import os

import numpy as np
import pytest

from oracle import ref_env

pytestmark = pytest.mark.gpu

REF = ref_env.install()
if REF is None:
    pytest.skip("reference tree not present (oracle/make_ref.py makes oracle/_ref)",
                allow_module_level=True)

import ngraph as rng  # noqa: E402
import ngraph.transformers as ngt  # noqa: E402
import ngraph_python_b200.ngraph_plugin as plugin  # noqa: E402,F401
from tests.flexsim import flex_tolerance  # noqa: E402
from tests.golden import cases  # noqa: E402

FIX = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "fixtures")
# flex16 leaves out what the reference's flex transformer does not run either (batch
# normalisation) and the cases whose outputs are whole parameter sets after optimizer steps
# (covered with their own bars in test_dp_gpu.py)
FLEX_SKIP = {"batchnorm_train", "mlp_train_step", "mlp_c1_train_step", "resnet_train_step",
             "reduce_4d_axis3", "softmax_xent", "unary_binary_sweep", "slice_views"}


def _as_list(res):
    return list(res) if isinstance(res, (tuple, list)) else [res]


def _run(factory_name, name, **kw):
    outs, params, vals = cases.CASES[name](rng)
    t = ngt.make_transformer_factory(factory_name, **kw)()
    comp = t.computation(outs, *params)
    results = []
    for rep in range(cases.REPEAT.get(name, 1)):
        results.append([np.array(r, copy=True) for r in _as_list(comp(*vals))])
    t.close()
    return results


@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_plugin_fp32_matches_cpu_transformer(name):
    want = _run("cpu", name)
    got = _run("b200", name)
    for rep, (g_rep, w_rep) in enumerate(zip(got, want)):
        for k, (g_, w_) in enumerate(zip(g_rep, w_rep)):
            assert g_.shape == w_.shape, (name, k)
            atol = 1e-5 * max(1.0, float(np.max(np.abs(w_))))
            np.testing.assert_allclose(g_, w_, rtol=1e-4, atol=atol,
                                       err_msg="%s output %d call %d" % (name, k, rep))
    # the committed fixture was made by the same CPU transformer elsewhere: same numbers here
    fix = np.load(os.path.join(FIX, name + ".npz"))
    for rep, w_rep in enumerate(want):
        for k, w_ in enumerate(w_rep):
            np.testing.assert_allclose(w_, fix["out%d_%d" % (rep, k)], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("name", sorted(set(cases.CASES) - FLEX_SKIP))
def test_plugin_flex16_within_reference_tolerance(name):
    want = _run("cpu", name)
    got = _run("b200", name, flex=True)
    for rep, (g_rep, w_rep) in enumerate(zip(got, want)):
        for k, (g_, w_) in enumerate(zip(g_rep, w_rep)):
            atol, rtol = flex_tolerance(w_)
            np.testing.assert_allclose(g_, w_, rtol=rtol, atol=4 * atol,
                                       err_msg="%s output %d call %d" % (name, k, rep))


def _reference_resnet20(n):
    """examples/resnet/resnet.py:74-117 of the reference, as the benchmark names it: CIFAR-10
    ResNet-20 (3 residual modules per stage), batch norm folded away, inference mode."""
    from resnet import BuildResnet
    from ngraph.frontends.neon import ax, Layer
    ax.N.length = n
    ax.Y.length = 10
    C, H, W = rng.make_axis(3, name="C"), rng.make_axis(32, name="H"), rng.make_axis(32, name="W")
    x = rng.placeholder([C, H, W, ax.N])
    np.random.seed(0)
    model = BuildResnet('cifar10', 20, False, 3, batch_norm=False)
    from ngraph.frontends.neon import Sequential
    with Layer.inference_mode_on():
        out = model(x)
        # without batch norm the softmax of this network is all but one-hot; the pooled features
        # under the linear layer (same layers, same weights) are what the comparison bites on
        feat = Sequential(model.layers[:-2])(x)
    xv = np.random.RandomState(100).uniform(0, 255, (3, 32, 32, n)).astype(np.float32)
    return [out, feat], x, xv


@pytest.mark.parametrize("flex", [True, False])
def test_reference_resnet20_batch_256(flex):
    """The benchmarked configuration itself: the reference's ResNet-20 builder at batch 256,
    through the plug-in on the device, against the reference CPU transformer on the same graph
    and input.  flex16: every convolution must run on the byte-plane tile kernel and every 3x3
    layer must carry its ReLU / residual tail in that kernel's epilogue -- the path the benchmark
    times."""
    out, x, xv = _reference_resnet20(256)
    cpu = ngt.make_transformer_factory("cpu")()
    want = [np.array(r, copy=True) for r in cpu.computation(out, x)(xv)]
    cpu.close()
    t = ngt.make_transformer_factory("b200", flex=flex)()
    comp = t.computation(out, x)
    got = [[np.array(r, copy=True) for r in comp(xv)] for _ in range(2)]
    convs = [s for s in comp.impl.steps if s.kind == "conv"]
    assert len(convs) == 44        # the network twice: once under the softmax, once for the features
    if flex:
        assert all(s.use_planes for s in convs)
        assert all(s.epi for s in convs if s.dims.R == 3)
    comp.impl.capture()                        # and as the replayed CUDA graph the benchmark times
    got.append([np.array(r, copy=True) for r in comp(xv)])
    t.close()
    assert want[0].shape == (10, 256) and want[1].size == 64 * 256
    assert float(np.abs(want[1]).max()) > 1.0          # the features are not degenerate
    for res in got:
        for g_, w_ in zip(res, want):
            g_ = g_.reshape(w_.shape)
            if flex:
                atol, rtol = flex_tolerance(w_)
                np.testing.assert_allclose(g_, w_, rtol=rtol, atol=4 * atol)
            else:
                np.testing.assert_allclose(g_, w_, rtol=1e-4,
                                           atol=1e-5 * max(1.0, float(np.abs(w_).max())))
        assert (res[0].argmax(axis=0) == want[0].argmax(axis=0)).mean() >= 0.97
    if not flex:
        assert all(np.array_equal(a, b) for a, b in zip(got[1], got[2]))
