"""Host logic without a GPU: graph building, fusion decisions and program generation (every
planned kernel is compiled for sm_100a by NVRTC), checked on the shared graph cases."""
import numpy as np
import pytest

import ngraph_python_b200 as ng
from ngraph_python_b200 import lib
from tests.golden import cases


def _plan(name, flex=False):
    outs, params, vals = cases.CASES[name](ng)
    t = ng.transformers.allocate_transformer("b200", plan_only=True, flex=flex)
    comp = t.computation(outs, *params)
    t.initialize()
    return t, comp


@pytest.mark.parametrize("flex", [False, True])
@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_every_case_plans_and_compiles(name, flex):
    t, comp = _plan(name, flex)
    assert len(comp.steps) >= 1
    for s in comp.steps:
        if s.kind == "ew":
            assert "b2_ew_main" in s.kernel.source()
        else:
            assert s.kind in ("gemm", "conv", "conv_bprop", "conv_update", "pool", "comm") and s.launches >= 0


def test_c2_is_one_kernel():
    """The whole microbenchmark graph (11 ops in the reference, one launch each) is one launch:
    4 loads, 1 elementwise store, 2 row reductions."""
    t, comp = _plan("c2_fused")
    assert len(comp.steps) == 1
    p = comp.steps[0].kernel.prog
    assert (p.n_in, p.n_out, p.n_red) == (4, 1, 2)
    assert p.reduce_mode == lib.REDUCE_C
    assert (p.A, p.B, p.C) == (1, 24, 2048)
    with pytest.raises(lib.B200Error):
        comp(*[np.zeros((24, 2048), np.float32)] * 4)


def test_softmax_splits_at_reductions():
    """A value needed only after a whole reduction starts a new kernel (the reference's stage
    boundary, ngraph/transformers/gpu/float_ew2.py:553-612)."""
    t, comp = _plan("softmax_xent")
    assert 3 <= len(comp.steps) <= 5


def test_inplace_update_stays_ordered():
    """A reader of a tensor that the same kernel has just assigned takes the value from the
    register of the assignment.  flex16: through a requant op that refers to the stored result,
    so that it sees the quantised value a later kernel would load."""
    t, comp = _plan("assign_sequence", flex=False)
    assert len(comp.steps) == 1
    prog = comp.steps[0].kernel.prog
    assert all(prog.ops[i].opcode != lib.OPCODES["requant"] for i in range(prog.n_ops))
    t, comp = _plan("assign_sequence", flex=True)
    assert len(comp.steps) == 1
    prog = comp.steps[0].kernel.prog
    rq = [prog.ops[i] for i in range(prog.n_ops) if prog.ops[i].opcode == lib.OPCODES["requant"]]
    assert len(rq) >= 1
    for op in rq:
        assert 0 <= op.b < prog.n_out and prog.out[op.b].t.dtype == lib.FLEX16
    src = comp.steps[0].kernel.source()
    assert "b2_requant(" in src


def test_broadcast_by_axis_name():
    K, N = ng.make_axis(3, name="K"), ng.make_axis(5, name="N")
    x, b = ng.placeholder([K, N]), ng.placeholder([N])
    assert (x + b).axes == ng.make_axes([K, N])
    assert (b + x).axes == ng.make_axes([N, K])
    assert ng.sum(x, reduction_axes=[K]).axes == ng.make_axes([N])
    with pytest.raises(ValueError):
        ng.sum(b, reduction_axes=[K])
    with pytest.raises(ValueError):
        ng.make_axes([K, K])


def test_api_errors_match_reference_wording():
    t = ng.transformers.allocate_transformer("b200", plan_only=True)
    x = ng.placeholder([ng.make_axis(4, name="A")])
    c = t.computation(ng.tanh(x), x)
    t.initialize()
    with pytest.raises(ValueError, match="finalized"):
        t.computation(ng.exp(x), x)
    with pytest.raises(ValueError, match="invalid/unsupported"):
        ng.transformers.allocate_transformer("nope")
    assert "b200" in ng.transformers.transformer_choices()


def test_no_cpu_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("device present")
    with pytest.raises(ng.UnsupportedTransformerException):
        ng.transformers.make_transformer()


def test_resnet20_plan_shape():
    """22 convolutions, one pooling, one dot; everything between them fused."""
    t, comp = _plan("resnet20")
    kinds = [s.kind for s in comp.steps]
    assert kinds.count("conv") == 22
    assert kinds.count("pool") == 1
    assert kinds.count("gemm") == 1
    # bias/ReLU/residual chains collapse: far fewer elementwise kernels than the 60+ ops
    assert kinds.count("ew") <= 26


def test_reduction_of_a_tensor_assigned_in_the_same_kernel():
    """fp32: a reduction that reads a persistent tensor right after its assignment takes the
    assigned value from the kernel's registers (the GEMM bench graph has this shape)."""
    A, B = ng.make_axis(6, name="A"), ng.make_axis(5, name="B")
    x = ng.placeholder([A, B])
    keep = ng.persistent_tensor([A, B])
    out = ng.sequential([ng.assign(keep, x * 2.0), ng.max(keep, reduction_axes=[A])])
    t = ng.transformers.allocate_transformer("b200", plan_only=True)
    comp = t.computation(out, x)
    t.initialize()
    assert len(comp.steps) == 1
