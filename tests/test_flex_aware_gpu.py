"""Flex-aware evaluation of whole graphs: every tensor the device stores is within ONE mantissa
step of what the graph's arithmetic gives for it.

After a computation has run in flex16, every stored tensor of the graph is read back as it lies
on the device -- int16 mantissas (or the two byte planes a convolution leaves for the next one)
and the exponent they were written with.  Each tensor is then recomputed on the host from the
stored values of the tensors it is computed from (the ops between two stored tensors -- a fused
kernel, a convolution with its bias / residual / ReLU tail -- in floating point, as the device
does), quantised with the exponent the device used for it, and compared mantissa by mantissa.

Because every tensor is recomputed from what the device really holds for its inputs, a difference
cannot grow from layer to layer, and the bar is the format's own: one step (rounding of a value
that lies within floating-point error of a half step).  The reference's flex tests hold single ops
to exact values (tests/flex_tests/test_flexew, run unchanged by tests/reference_suite.py); this
holds whole networks -- 22 convolution layers through the implicit-GEMM kernels, pooling,
classifier, softmax, and the gradient contractions -- to the same granularity.
"""
import numpy as np
import pytest

from tests.golden import cases
from tests.mirror_interp import Interp

pytestmark = pytest.mark.gpu


def _mantissas(t, buf):
    """int64 mantissas of a flex16 buffer as the device holds them (flat, buffer order)."""
    if buf.planes_by_producer:
        # written as two byte planes only: high bytes (signed) then low bytes (unsigned)
        off = buf.planes_ptr - buf.planes.data_ptr()
        raw = buf.planes.cpu().numpy()
        hi = raw[off:off + buf.size].view(np.int8).astype(np.int64)
        lo = raw[off + buf.plane_bytes:off + buf.plane_bytes + buf.size].astype(np.int64)
        return hi * 256 + lo
    return buf.tensor.cpu().numpy()[:buf.size].astype(np.int64)


def _stored(t, comp):
    """{op: (view, mantissas, step)} for every op whose value a kernel of `comp` stored in a
    buffer of its own, plus the computation's inputs and variables."""
    from ngraph_python_b200.op_graph import AssignableTensorOp
    # (out_views, not output_buffers(): a pooling result shares its input's exponent entry and is
    # not listed as a separately managed buffer, but it is stored all the same)
    written = set(id(v.buffer) for s in comp.steps for v in s.out_views)
    out = {}
    for op, view in t._views.items():
        buf = view.buffer
        if not buf.flex or not view.is_dense() or view.offset != 0 or \
                tuple(view.axes.lengths) != tuple(buf.axes.lengths):
            continue            # a window on somebody else's storage
        if id(buf) in written or isinstance(op, AssignableTensorOp):
            out.setdefault(id(buf), (op, view, buf))
    res = {}
    for op, view, buf in out.values():
        step = float(t._table_np[buf.slot, 0])
        res[op] = (view, _mantissas(t, buf), step, id(buf))
    return res


def _value(view, mant, step, op):
    """The stored tensor as floats in the op's own axis order."""
    arr = (mant.astype(np.float64) * step).reshape(view.axes.lengths)
    names = [a.name for a in view.axes]
    perm = [names.index(a.name) for a in op.axes]
    return np.ascontiguousarray(np.transpose(arr, perm)).astype(np.float32)


def _check(t, comp, min_checked):
    from ngraph_python_b200.op_graph import AssignableTensorOp
    stored = _stored(t, comp)
    values = {op: _value(v, m, s, op) for op, (v, m, s, _) in stored.items()}
    # a kernel that stores several tensors computes each of them from the floating-point values
    # of the others, not from what it stored of them: only tensors of OTHER kernels are given
    siblings = {}
    for s in comp.steps:
        ids = set(id(v.buffer) for v in s.out_views)
        for i in ids:
            siblings[i] = ids
    checked, worst, failures = 0, 0, []
    for op, (view, mant, step, buf_id) in stored.items():
        if isinstance(op, AssignableTensorOp):
            continue
        it = Interp()
        for other, val in values.items():
            if stored[other][3] in siblings.get(buf_id, (buf_id,)):
                continue
            if isinstance(other, AssignableTensorOp):
                it.state[other] = val
            else:
                it.cache[other] = val
        want = np.asarray(it.eval(op), dtype=np.float64)
        names = [a.name for a in op.axes]
        perm = [names.index(a.name) for a in view.axes]
        want = np.transpose(want.reshape(op.axes.lengths), perm).reshape(-1)
        m_want = np.clip(np.rint(want / step), -32768, 32767).astype(np.int64)
        diff = np.abs(m_want - mant)
        worst = max(worst, int(diff.max()))
        if diff.max() > 1:
            failures.append("%s: %d of %d mantissas off by more than one step (max %d, step %g, "
                            "largest mantissa %d)" % (op, int((diff > 1).sum()), diff.size,
                                                      int(diff.max()), step, int(np.abs(mant).max())))
        elif (diff > 0).mean() >= 0.05:
            # a one-step difference is rounding at a half step, not an offset: rare
            failures.append("%s: %.1f %% of the mantissas differ by a step (step %g)" % (
                op, 100.0 * (diff > 0).mean(), step))
        checked += 1
    assert not failures, "\n".join(failures)
    assert checked >= min_checked, "only %d stored tensors were checked" % checked
    return checked, worst


def _run(ng, builder, calls=3, **kw):
    outs, params, vals = builder(ng, **kw)
    t = ng.transformers.allocate_transformer("b200", flex=True)
    comp = t.computation(outs, *params)
    for _ in range(calls):
        comp(*vals)             # exponents settle on the data (the inputs do not change)
    return t, comp


def test_resnet20_every_stored_tensor_within_one_step():
    """ResNet-20 at a batch the tile kernels take (128 images, 32x32): the input planes, 22
    convolution layers with their tails, pooling, classifier, softmax."""
    import ngraph_python_b200 as ng
    from ngraph_python_b200 import configs
    t, comp = _run(ng, configs.resnet20, n=128, hw=32)
    assert all(s.use_planes for s in comp.steps if s.kind == "conv")
    checked, _ = _check(t, comp, min_checked=24)
    t.close()


def test_resnet8_gather_path_every_stored_tensor_within_one_step():
    """The same network family at a batch the tile kernels do not take (32 images): gather + GEMM."""
    import ngraph_python_b200 as ng
    t, comp = _run(ng, cases.resnet8_small)
    _check(t, comp, min_checked=8)
    t.close()


@pytest.mark.parametrize("case,kw", [("conv_grads", dict(N=128)), ("conv_grads_stride2", {}),
                                     ("mlp_forward", {}), ("softmax_xent", {}),
                                     ("pool_grads", {}), ("c2_fused", {})])
def test_graph_cases_every_stored_tensor_within_one_step(case, kw):
    import ngraph_python_b200 as ng
    t, comp = _run(ng, cases.CASES[case] if hasattr(cases, "CASES") else getattr(cases, case), **kw)
    _check(t, comp, min_checked=1)
    t.close()
