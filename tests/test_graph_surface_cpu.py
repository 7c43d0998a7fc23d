"""The graph-building surface on CPU: every shared case, built with ngraph_python_b200 and
evaluated by the numpy interpreter of tests/mirror_interp.py, must reproduce the fixtures made
by the reference's CPU transformer -- axes algebra, broadcasting by axis name, dot contraction,
views and sequential/assign ordering all take part."""
import os

import numpy as np
import pytest

import ngraph_python_b200 as ng
from tests.golden import cases
from tests.mirror_interp import Interp

FIX = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "fixtures")


@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_mirror_graph_matches_reference_cpu(name):
    fix = np.load(os.path.join(FIX, name + ".npz"))
    outs, params, vals = cases.CASES[name](ng)
    it = Interp()
    for rep in range(cases.REPEAT.get(name, 1)):
        res = it.run(outs, dict(zip(params, vals)))
        for k, got in enumerate(res):
            exp = fix["out%d_%d" % (rep, k)]
            assert got.shape == exp.shape
            atol = 2e-5 * max(1.0, float(np.max(np.abs(exp))))
            np.testing.assert_allclose(got, exp, rtol=2e-4, atol=atol,
                                       err_msg="%s output %d call %d" % (name, k, rep))
