"""The reference's flex golden vectors through the real device path: flex transformer with one
kernel per op (the reference's execution model), scalar and small-array operands, exponent
management on the host, quantise/saturate/statistics on the GPU."""
import numpy as np
import pytest

import ngraph_python_b200 as ng
from tests.flexsim import flex_tolerance
from tests.golden.flex_vectors import CASES

pytestmark = pytest.mark.gpu

UNARY = {"neg": ng.negative, "sqrt": ng.sqrt, "abs": ng.absolute, "exp": ng.exp, "log": ng.log,
         "safelog": ng.safelog, "tanh": ng.tanh, "rcp": ng.reciprocal, "sqr": ng.square,
         "sig": ng.sigmoidAtomic, "sigmoid_composed": ng.sigmoid}
BINARY = {"add": ng.add, "sub": ng.subtract, "mul": ng.multiply, "div": ng.divide, "mod": ng.mod,
          "pow": ng.power, "maximum": ng.maximum, "minimum": ng.minimum, "eq": ng.equal,
          "ne": ng.not_equal, "lt": ng.less, "le": ng.less_equal, "gt": ng.greater,
          "ge": ng.greater_equal}
REDUCE = {"sum": ng.sum, "prod": ng.prod, "max": ng.max, "min": ng.min, "argmax": ng.argmax,
          "argmin": ng.argmin}


def _placeholder_like(v):
    v = np.asarray(v)
    axes = [ng.make_axis(n) for n in v.shape]
    return ng.placeholder(axes), axes


def _build(op, first_operands):
    ph, axes = _placeholder_like(first_operands[0])
    if op == "assign_var":
        var = ng.variable(())
        return ng.sequential([ng.assign(var, ph), var]), [ph]
    if op in UNARY:
        return UNARY[op](ph), [ph]
    if op in REDUCE:
        return REDUCE[op](ph, reduction_axes=axes), [ph]
    ph2 = ng.placeholder(axes)
    return BINARY[op](ph, ph2), [ph, ph2]


# libm-dependent single-call vectors: CUDA's expf/logf/powf may differ from the reference GPU's
# by an ulp, which can move a mantissa by one unit; they are compared to one mantissa step.
@pytest.mark.parametrize("case", CASES, ids=lambda c: "%s@%s" % (c[0], c[2].split("/")[-1]))
def test_golden_vector_on_device(case):
    op, calls, src = case
    graph, params = _build(op, calls[0][0])
    t = ng.transformers.allocate_transformer("b200", flex=True, fuse=False)
    comp = t.computation(graph, *params)
    iterations = len(calls) != 1
    for operands, expected in calls:
        got = comp(*[np.asarray(o, dtype=np.float64) for o in operands])
        expected = np.asarray(expected, dtype=np.float64)
        if iterations:
            atol, rtol = flex_tolerance(expected)
            np.testing.assert_allclose(got, expected, rtol=rtol, atol=atol,
                                       err_msg="%s %s" % (src, operands))
        elif op in ("exp", "log", "safelog", "pow", "tanh", "sig", "sigmoid_composed", "sqrt"):
            out_buf = comp.return_views[0].buffer
            step = out_buf.entry.scale
            assert np.all(np.abs(np.asarray(got) - expected) <= step), \
                "%s %s: got %r expected %r" % (src, operands, got, expected)
        else:
            assert np.array_equal(np.asarray(got, dtype=np.float64), expected), \
                "%s %s: got %r expected %r" % (src, operands, got, expected)
    t.close()
