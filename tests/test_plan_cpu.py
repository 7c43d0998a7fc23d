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
            assert s.kind in ("gemm", "conv", "conv_bprop", "conv_update", "pool", "pool_bprop",
                              "lut", "lut_update", "comm") and s.launches >= 0


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


def test_plane_entry_points_describe_the_dilated_error_tensor():
    """Host arithmetic of the C ABI (no device): the input gradient of a strided convolution
    streams the error tensor zero-dilated to H+2pad-R+1 rows; strides whose zero filling would
    multiply the work by more than four stay on the gather path."""
    import ctypes as C

    def dims(Cc, H, W, N, K, R, S, pad, stride):
        d = lib.ConvDims()
        P, Q = (H + 2 * pad - R) // stride + 1, (W + 2 * pad - S) // stride + 1
        for k, v in dict(C=Cc, D=1, H=H, W=W, N=N, K=K, T=1, R=R, S=S, M=1, P=P, Q=Q, pad_d=0,
                         pad_h=pad, pad_w=pad, str_d=1, str_h=stride, str_w=stride, dil_d=1,
                         dil_h=1, dil_w=1).items():
            setattr(d, k, v)
        return d, P, Q
    d, P, Q = dims(16, 32, 32, 128, 32, 3, 3, 1, 2)
    ok, act, filt = lib.conv_planes_info(d, lib.CONV_BPROP)
    assert ok and act == (32 * 32 * 32 * 128 + 1023) // 1024 * 1024      # K x (H+2-3+1)^2 x N
    ok1, act1, _ = lib.conv_planes_info(dims(16, 32, 32, 128, 32, 3, 3, 1, 1)[0], lib.CONV_BPROP)
    assert ok1 and act1 == act                                            # unit stride: K x P x Q x N
    assert not lib.conv_planes_info(dims(16, 33, 33, 128, 32, 3, 3, 0, 3)[0], lib.CONV_BPROP)[0]
    assert not lib.conv_planes_info(dims(16, 32, 32, 96, 32, 3, 3, 1, 2)[0], lib.CONV_BPROP)[0]
    # filter gradient on the tile kernel: planes of both operands + int64 slices; far less than
    # the unrolled input the gather path writes
    small = lib.conv_update_scratch_bytes(True, dims(16, 32, 32, 128, 16, 3, 3, 1, 1)[0])
    odd_batch = lib.conv_update_scratch_bytes(True, dims(16, 32, 32, 96, 16, 3, 3, 1, 1)[0])
    assert small < odd_batch
