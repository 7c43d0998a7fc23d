"""The plug-in that registers the b200 transformer inside nGraph-Python itself.  Needs the
reference tree (skipped where it is absent): graphs are built with the REAL ngraph ops, go
through ngraph.transformers.make_transformer_factory('b200'), are translated to this package's
op surface and planned; the translated graphs are also evaluated with numpy and compared with
the fixtures that the reference CPU transformer produced for the same graphs."""
import os

import numpy as np
import pytest

from oracle import ref_env  # noqa: E402

REF = ref_env.install()
if REF is None:
    pytest.skip("reference tree not present (oracle/make_ref.py makes oracle/_ref)",
                allow_module_level=True)

HERE = os.path.dirname(os.path.abspath(__file__))
import ngraph as rng  # noqa: E402
import ngraph.transformers as ngt  # noqa: E402
import ngraph_python_b200.ngraph_plugin as plugin  # noqa: E402,F401
from tests.golden import cases  # noqa: E402
from tests.mirror_interp import Interp  # noqa: E402

FIX = os.path.join(HERE, "golden", "fixtures")
NAMES = [n for n in sorted(cases.CASES) if n not in ("resnet20",)]


def test_registered_in_reference_registry():
    assert "b200" in ngt.transformer_choices()
    t = ngt.make_transformer_factory("b200", plan_only=True)()
    assert type(t).__name__ == "B200NgraphTransformer"
    t.close()


def test_flex_transformer_with_the_reference_granularity_is_registered():
    """'b200flex' stands where the reference's 'flexgpu' stands: flex16 storage, every op's result
    stored (one kernel per op), the flex transformer's tolerances and keyword arguments
    (flexgputransform.py:67-103)."""
    assert "b200flex" in ngt.transformer_choices()
    t = ngt.make_transformer_factory("b200flex", plan_only=True, fixed_point=True)()
    assert t.impl.flex and not t.impl.fuse and t.impl.fixed_point
    atol, rtol = type(t).get_default_tolerance(np.array([100.0]))
    assert rtol == 1e-2 and atol == 8 * 2.0 ** -8          # 100 needs dec 8: one step is 2^-8
    A = rng.make_axis(4, name="A")
    x = rng.placeholder([A])
    comp = t.computation(rng.tanh(x) * 2.0 + x, x)
    t.initialize()
    assert len([s for s in comp.impl.steps if s.kind == "ew"]) == 3     # not fused into one
    t.close()


@pytest.mark.parametrize("flex", [False, True])
@pytest.mark.parametrize("name", NAMES)
def test_reference_graph_translates_and_plans(name, flex):
    outs, params, vals = cases.CASES[name](rng)
    t = ngt.make_transformer_factory("b200", plan_only=True, flex=flex)()
    comp = t.computation(outs, *params)
    t.initialize()
    assert len(comp.impl.steps) >= 1
    with pytest.raises(Exception):
        comp(*vals)          # planned only: no device here
    t.close()


@pytest.mark.parametrize("name", NAMES)
def test_translated_graph_matches_reference_cpu(name):
    fix = np.load(os.path.join(FIX, name + ".npz"))
    outs, params, vals = cases.CASES[name](rng)
    tr = plugin.GraphTranslator()
    m_outs = [tr(o) for o in outs]
    m_params = [tr(p) for p in params]
    it = Interp()
    for rep in range(cases.REPEAT.get(name, 1)):
        res = it.run(m_outs, dict(zip(m_params, vals)))
        for k, got in enumerate(res):
            exp = fix["out%d_%d" % (rep, k)]
            atol = 2e-5 * max(1.0, float(np.max(np.abs(exp))))
            np.testing.assert_allclose(got.reshape(exp.shape), exp, rtol=2e-4, atol=atol,
                                       err_msg="%s output %d call %d" % (name, k, rep))


def test_neon_model_with_reference_autodiff_and_optimizer():
    """A small convolutional network built with the reference's neon frontend, differentiated by
    the reference's autodiff and updated by its GradientDescentMomentum: the translated graph
    (pooling and convolution gradients, slices and their adjoints, control dependencies, one-hot
    targets) plans for the device, and evaluated with numpy it follows the reference CPU
    transformer through three training steps."""
    from ngraph.frontends.neon import (Sequential, Convolution, Pooling, Affine, Rectlin, Softmax,
                                       GaussianInit, ConstantInit, GradientDescentMomentum, ax)
    ax.N.length = 32
    ax.Y.length = 10
    C, D = rng.make_axis(3, name="C"), rng.make_axis(1, name="D")
    H, W = rng.make_axis(16, name="H"), rng.make_axis(16, name="W")
    x = rng.placeholder([C, D, H, W, ax.N])
    t = rng.placeholder([ax.N])
    init = GaussianInit(0., 0.1)
    model = Sequential([
        Convolution((3, 3, 8), filter_init=init, strides=1, padding=1, activation=Rectlin()),
        Pooling((2, 2), strides=2, pool_type="max"),
        Convolution((3, 3, 16), filter_init=init, strides=2, padding=1, activation=Rectlin()),
        Pooling((2, 2), strides=2, pool_type="avg"),
        Affine(weight_init=init, bias_init=ConstantInit(0.), activation=Softmax(), axes=(ax.Y,))])
    loss = rng.cross_entropy_multi(model(x), rng.one_hot(t, axis=ax.Y))
    updates = GradientDescentMomentum(0.1, 0.9)(loss)
    train = rng.sequential([updates, rng.mean(loss, out_axes=[])])
    for flex in (False, True):
        tr = ngt.make_transformer_factory("b200", plan_only=True, flex=flex)()
        comp = tr.computation(train, x, t)
        tr.initialize()
        kinds = [s.kind for s in comp.impl.steps]
        assert kinds.count("conv") == 2 and kinds.count("conv_update") == 2
        assert kinds.count("conv_bprop") == 1 and kinds.count("pool_bprop") == 2
        assert kinds.count("gemm") == 3
        tr.close()
    rs = np.random.RandomState(3)
    xv = rs.standard_normal((3, 1, 16, 16, 32)).astype(np.float32)
    tv = rs.randint(0, 10, 32).astype(np.float32)
    cpu = ngt.make_transformer_factory("cpu")()
    cref = cpu.computation(train, x, t)
    want = [float(cref(xv, tv)) for _ in range(3)]
    cpu.close()
    trn = plugin.GraphTranslator()
    m_train, m_x, m_t = trn(train), trn(x), trn(t)
    it = Interp()
    got = [float(np.asarray(it.run([m_train], {m_x: xv, m_t: tv})[0])) for _ in range(3)]
    assert want[2] < want[0]                      # it does train
    np.testing.assert_allclose(got, want, rtol=2e-5)


def _reference_resnet(train):
    """The reference's own CIFAR-10 ResNet builder (examples/resnet/resnet.py: BuildResnet), 8
    layers, without batch normalisation -- the network of the headline benchmark, built by the
    reference's code rather than by this package's restatement of it."""
    from resnet import BuildResnet
    from ngraph.frontends.neon import ax, GradientDescentMomentum, Layer
    n = 32 if train else 128         # (128 images: the convolutions can run on the tile kernel)
    ax.N.length = n
    ax.Y.length = 10
    C, H, W = rng.make_axis(3, name="C"), rng.make_axis(32, name="H"), rng.make_axis(32, name="W")
    x = rng.placeholder([C, H, W, ax.N])
    t = rng.placeholder([ax.N])
    np.random.seed(0)
    model = BuildResnet('cifar10', 8, False, 1, batch_norm=False)
    rs = np.random.RandomState(1)
    xv = rs.uniform(0, 255, (3, 32, 32, n)).astype(np.float32)
    tv = rs.randint(0, 10, n).astype(np.float32)
    if not train:
        with Layer.inference_mode_on():
            return model(x), [x], [xv]
    loss = rng.cross_entropy_multi(model(x), rng.one_hot(t, axis=ax.Y))
    updates = GradientDescentMomentum(0.01, 0.9)(loss)
    return rng.sequential([updates, rng.mean(loss, out_axes=[])]), [x, t], [xv, tv]


@pytest.mark.parametrize("train", [False, True])
def test_reference_resnet_builder(train):
    """Inference: the layers' bias / ReLU / residual tails fold into the convolution steps in
    flex16.  Training: every convolution gets its filter gradient, all but the first their input
    gradient, from the ops the reference's autodiff created.  Both: the translated graph, evaluated
    with numpy, agrees with the reference CPU transformer."""
    out, params, vals = _reference_resnet(train)
    for flex in (False, True):
        tr = ngt.make_transformer_factory("b200", plan_only=True, flex=flex)()
        comp = tr.computation(out, *params)
        tr.initialize()
        kinds = [s.kind for s in comp.impl.steps]
        assert kinds.count("conv") == 10 and kinds.count("pool") == 1
        if train:
            assert kinds.count("conv_update") == 10 and kinds.count("conv_bprop") == 9
            assert kinds.count("pool_bprop") == 1 and kinds.count("gemm") == 3
        else:
            assert kinds.count("gemm") == 1
            if flex:
                assert kinds.count("ew") <= 6          # tails folded into the convolutions
        tr.close()
    cpu = ngt.make_transformer_factory("cpu")()
    cref = cpu.computation(out, *params)
    reps = 3 if train else 1
    want = [np.array(cref(*vals), copy=True) for _ in range(reps)]
    cpu.close()
    trn = plugin.GraphTranslator()
    m_out = trn(out)
    m_params = [trn(p) for p in params]
    it = Interp()
    got = [np.asarray(it.run([m_out], dict(zip(m_params, vals)))[0]) for _ in range(reps)]
    for g_, w_ in zip(got, want):
        np.testing.assert_allclose(g_, w_, rtol=2e-5, atol=2e-6)


# ---- automatic gradient exchange (two gloo ranks on CPU) -------------------------------------
def _dp_model(n):
    """A small convolutional classifier with the reference's autodiff and momentum optimizer,
    built for a batch of n images; weights from the global numpy seed."""
    from ngraph.frontends.neon import (Sequential, Convolution, Pooling, Affine, Rectlin, Softmax,
                                       GaussianInit, ConstantInit, GradientDescentMomentum, ax)
    ax.N.length = n
    ax.Y.length = 10
    C, D = rng.make_axis(3, name="C"), rng.make_axis(1, name="D")
    H, W = rng.make_axis(8, name="H"), rng.make_axis(8, name="W")
    x = rng.placeholder([C, D, H, W, ax.N])
    t = rng.placeholder([ax.N])
    np.random.seed(5)
    init = GaussianInit(0., 0.1)
    model = Sequential([
        Convolution((3, 3, 8), filter_init=init, strides=1, padding=1, activation=Rectlin()),
        Pooling((2, 2), strides=2, pool_type="avg"),
        Affine(weight_init=init, bias_init=ConstantInit(0.), activation=Softmax(), axes=(ax.Y,))])
    loss = rng.cross_entropy_multi(model(x), rng.one_hot(t, axis=ax.Y))
    updates = GradientDescentMomentum(0.1, 0.9)(loss)
    return rng.sequential([updates, rng.mean(loss, out_axes=[])]), x, t


def _dp_data(global_n):
    rs = np.random.RandomState(8)
    return (rs.standard_normal((3, 1, 8, 8, global_n)).astype(np.float32),
            rs.randint(0, 10, global_n).astype(np.float32))


def _dp_rank(rank, world, port, global_n, steps, q):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n = global_n // world
        train, x, t = _dp_model(n)
        tr = plugin.GraphTranslator(replicas=world)
        m_train, m_x, m_t = tr(train), tr(x), tr(t)

        def allreduce(arr, func):
            buf = torch.from_numpy(arr.copy())
            dist.all_reduce(buf)
            return buf.numpy() / (world if func == "mean" else 1)
        it = Interp(allreduce=allreduce)
        xv, tv = _dp_data(global_n)
        lo, hi = rank * n, (rank + 1) * n
        losses = [float(np.asarray(it.run([m_train], {m_x: xv[..., lo:hi], m_t: tv[lo:hi]})[0]))
                  for _ in range(steps)]
        q.put((rank, losses, len(tr.exchanges), sorted(set(e.reduce_func
                                                           for e in tr.exchanges.values()))))
    finally:
        dist.destroy_process_group()


def test_gradient_exchange_is_inserted_from_reduce_func_tags():
    """Two replicas, each with half of the batch, built from the reference's own autodiff and
    optimizer with nothing written by hand: the translation puts one exchange on every gradient
    (tagged reduce_func='sum' by the reference, op_graph.py:4294-4297) where the untagged
    `/ batch_size` reads it, and the two replicas then train exactly like the reference CPU
    transformer on the whole batch: the mean of their post-step losses follows its loss."""
    import socket
    import torch.multiprocessing as mp
    global_n, steps, world = 16, 3, 2
    train, x, t = _dp_model(global_n)
    cpu = ngt.make_transformer_factory("cpu")()
    cref = cpu.computation(train, x, t)
    xv, tv = _dp_data(global_n)
    want = [float(cref(xv, tv)) for _ in range(steps)]
    cpu.close()
    # one replica: nothing is inserted
    solo = plugin.GraphTranslator()
    solo(train)
    assert not solo.exchanges
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_dp_rank, args=(r, world, port, global_n, steps, q))
             for r in range(world)]
    for p in procs:
        p.start()
    try:
        got = dict((r, (l_, n_, f_)) for r, l_, n_, f_ in (q.get(timeout=300) for _ in range(world)))
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    finally:
        for p in procs:
            if p.is_alive():
                p.terminate()
    for r in range(world):
        assert got[r][1] == 3          # filters, linear weights, bias: one per trainable tensor
        assert got[r][2] == ["mean"]   # sum over replicas, divided by their number (shards)
    mean_loss = np.mean([got[r][0] for r in range(world)], axis=0)
    np.testing.assert_allclose(mean_loss, want, rtol=2e-5)
    assert want[-1] < want[0]


def _hetr_style_model(global_n):
    """The way hetr scripts annotate a data-parallel graph: built on the GLOBAL batch, everything
    under ng.metadata(device_id=(...), parallel=ax.N)."""
    from ngraph.frontends.neon import (Sequential, Affine, Rectlin, Softmax, GaussianInit,
                                       ConstantInit, GradientDescentMomentum, ax)
    ax.N.length = global_n
    ax.Y.length = 10
    F = rng.make_axis(24, name="F")
    with rng.metadata(device="gpu", device_id=("0", "1"), parallel=ax.N):
        x = rng.placeholder([F, ax.N])
        t = rng.placeholder([ax.N])
        np.random.seed(6)
        init = GaussianInit(0., 0.2)
        model = Sequential([
            Affine(weight_init=init, bias_init=ConstantInit(0.), activation=Rectlin(), nout=16),
            Affine(weight_init=init, bias_init=ConstantInit(0.), activation=Softmax(), axes=(ax.Y,))])
        probs = model(x)
        loss = rng.cross_entropy_multi(probs, rng.one_hot(t, axis=ax.Y))
        updates = GradientDescentMomentum(0.1, 0.9)(loss)
        train = rng.sequential([updates, probs])
    return train, x, t


def _hetr_rank(rank, world, port, global_n, steps, q):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        train, x, t = _hetr_style_model(global_n)
        tr = plugin.GraphTranslator(replicas=world, rank=rank)
        tr.set_parallel_axis(plugin._find_parallel_axis(rng.computation(train, x, t)))
        m_train, m_x, m_t = tr(train), tr(x), tr(t)
        assert m_x.axes.lengths == (24, global_n // world)

        def allreduce(arr, func):
            buf = torch.from_numpy(arr.copy())
            dist.all_reduce(buf)
            return buf.numpy() / (world if func == "mean" else 1)
        it = Interp(allreduce=allreduce)
        rs = np.random.RandomState(9)
        xv = rs.standard_normal((24, global_n)).astype(np.float32)
        tv = rs.randint(0, 10, global_n).astype(np.float32)
        n = global_n // world
        lo, hi = rank * n, (rank + 1) * n
        outs = [np.asarray(it.run([m_train], {m_x: xv[:, lo:hi], m_t: tv[lo:hi]})[0])
                for _ in range(steps)]
        q.put((rank, outs, sorted(set(e.reduce_func for e in tr.exchanges.values()))))
    finally:
        dist.destroy_process_group()


def test_hetr_style_graph_runs_as_shards():
    """A graph annotated for hetr -- global batch, ng.metadata(device_id=(...), parallel=ax.N) --
    is cut along the parallel axis per replica: placeholders shrink to the replica's share,
    gradients are summed over the replicas (the optimizer already divides by the global batch)
    and the replicas' outputs, put side by side, are the reference CPU transformer's on the whole
    batch, step after step."""
    import socket
    import torch.multiprocessing as mp
    global_n, steps, world = 16, 3, 2
    train, x, t = _hetr_style_model(global_n)
    assert plugin._find_parallel_axis(rng.computation(train, x, t)).length == global_n
    cpu = ngt.make_transformer_factory("cpu")()
    cref = cpu.computation(train, x, t)
    rs = np.random.RandomState(9)
    xv = rs.standard_normal((24, global_n)).astype(np.float32)
    tv = rs.randint(0, 10, global_n).astype(np.float32)
    want = [np.array(cref(xv, tv), copy=True) for _ in range(steps)]
    cpu.close()
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_hetr_rank, args=(r, world, port, global_n, steps, q))
             for r in range(world)]
    for p in procs:
        p.start()
    try:
        got = dict((r, (o, f)) for r, o, f in (q.get(timeout=300) for _ in range(world)))
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
    finally:
        for p in procs:
            if p.is_alive():
                p.terminate()
    assert got[0][1] == ["sum"] and got[1][1] == ["sum"]
    for k in range(steps):
        whole = np.concatenate([got[0][0][k], got[1][0][k]], axis=1)
        np.testing.assert_allclose(whole, want[k], rtol=2e-5, atol=1e-6)
