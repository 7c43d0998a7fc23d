"""The plug-in that registers the b200 transformer inside nGraph-Python itself.  Needs the
reference tree (skipped where it is absent): graphs are built with the REAL ngraph ops, go
through ngraph.transformers.make_transformer_factory('b200'), are translated to this package's
op surface and planned; the translated graphs are also evaluated with numpy and compared with
the fixtures that the reference CPU transformer produced for the same graphs."""
import os
import sys

import numpy as np
import pytest

REF = "/root/reference"
if not os.path.isdir(os.path.join(REF, "ngraph")):
    pytest.skip("reference tree not present", allow_module_level=True)

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden", "ref_shims"))
import ref_bootstrap  # noqa: E402

ref_bootstrap.install(REF)
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
