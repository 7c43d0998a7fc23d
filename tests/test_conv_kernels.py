"""GPU parity of the convolution / pooling entry points through the C ABI.

flex16 with small integer data must equal the exact integer convolution (the reference's own
flex convolution test asserts np.array_equal on integer inputs in [-4, 4):
tests/flex_tests/test_flexconv.py:60-70); full-range mantissas are checked against the int64
oracle with the exact round-to-nearest-even rescale."""
import ctypes as C

import numpy as np
import pytest

from oracle import conv_oracle as co

pytestmark = pytest.mark.gpu

# (C, H, W, N, K, R, S, pad, stride): shapes of the reference's flex conv tests plus ResNet-20's
SHAPES = [(16, 7, 7, 32, 8, 3, 3, 0, 1), (16, 9, 11, 32, 8, 3, 3, 1, 1), (3, 32, 32, 32, 16, 3, 3, 1, 1),
          (16, 16, 16, 64, 32, 3, 3, 1, 2), (32, 16, 16, 32, 64, 1, 1, 0, 2), (64, 8, 8, 32, 64, 3, 3, 1, 1),
          (5, 6, 5, 24, 10, 2, 3, 1, 1),
          # batches that are a multiple of 128 take the implicit-GEMM kernel
          (16, 8, 8, 128, 16, 3, 3, 1, 1), (3, 10, 9, 128, 16, 3, 3, 1, 1), (16, 12, 12, 256, 32, 3, 3, 1, 2),
          (32, 8, 8, 128, 64, 1, 1, 0, 2), (64, 6, 6, 128, 64, 3, 3, 1, 1), (40, 5, 7, 128, 24, 3, 2, 1, 1),
          (16, 6, 6, 128, 144, 3, 3, 1, 1)]


def _dims(lib, Cc, H, W, N, K, R, S, pad, stride):
    d = lib.ConvDims()
    P = (H + 2 * pad - R) // stride + 1
    Q = (W + 2 * pad - S) // stride + 1
    d.C, d.D, d.H, d.W, d.N = Cc, 1, H, W, N
    d.K, d.T, d.R, d.S = K, 1, R, S
    d.M, d.P, d.Q = 1, P, Q
    d.pad_d, d.pad_h, d.pad_w = 0, pad, pad
    d.str_d, d.str_h, d.str_w = 1, stride, stride
    d.dil_d = d.dil_h = d.dil_w = 1
    return d, P, Q


def _scratch(torch, nbytes):
    t = torch.empty((nbytes + 1024,), dtype=torch.uint8, device="cuda")
    return t, t.data_ptr() + (-t.data_ptr()) % 1024


@pytest.mark.parametrize("shape", SHAPES)
def test_conv_fprop_f32(shape):
    import torch
    from ngraph_python_b200 import lib
    Cc, H, W, N, K, R, S, pad, stride = shape
    d, P, Q = _dims(lib, *shape)
    rng = np.random.RandomState(sum(shape))
    I = rng.standard_normal((Cc, H, W, N)).astype(np.float32)
    F = rng.standard_normal((Cc, R, S, K)).astype(np.float32)
    dI, dF = torch.from_numpy(I).cuda(), torch.from_numpy(F).cuda()
    dO = torch.zeros((K, P, Q, N), dtype=torch.float32, device="cuda")
    status = torch.zeros((1,), dtype=torch.int32, device="cuda")
    nb = lib.conv_fprop_scratch_bytes(False, d)
    keep, sp = _scratch(torch, nb)
    lib.check(lib.raw().b2_conv_fprop_f32(dI.data_ptr(), dF.data_ptr(), dO.data_ptr(), C.byref(d),
                                          sp, nb, status.data_ptr(), 0))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    exp = co.conv_fprop(I, F, (pad, pad), (stride, stride), dtype=np.float64)
    np.testing.assert_allclose(dO.cpu().numpy(), exp, rtol=1e-4, atol=1e-5 * np.sqrt(Cc * R * S) * 4)


@pytest.mark.parametrize("small", [True, False])
@pytest.mark.parametrize("shape", SHAPES)
def test_conv_fprop_flex16_exact(shape, small):
    import torch
    from ngraph_python_b200 import lib
    Cc, H, W, N, K, R, S, pad, stride = shape
    d, P, Q = _dims(lib, *shape)
    rng = np.random.RandomState(sum(shape) + 1)
    lim = 4 if small else 32767
    I = rng.randint(-lim, lim, (Cc, H, W, N)).astype(np.int16)
    F = rng.randint(-lim, lim, (Cc, R, S, K)).astype(np.int16)
    exact = co.conv_fprop(I, F, (pad, pad), (stride, stride), dtype=np.int64)
    # small integers: all exponents 0, the output mantissas ARE the integer convolution
    dec_i = dec_f = 0
    sh = 0 if small else max(0, int(np.ceil(np.log2(max(1, np.abs(exact).max()) / 32767.0))) + 1)
    dec_o = dec_i + dec_f - sh
    dI, dF = torch.from_numpy(I).cuda(), torch.from_numpy(F).cuda()
    dO = torch.zeros((K, P, Q, N), dtype=torch.int16, device="cuda")
    table = torch.tensor([[1.0, 1.0], [1.0, 1.0], [2.0 ** -dec_o, 2.0 ** dec_o]],
                         dtype=torch.float32, device="cuda")
    stats = torch.zeros((3,), dtype=torch.int32, device="cuda")
    probe = torch.zeros((1,), dtype=torch.int64, device="cuda")
    status = torch.zeros((1,), dtype=torch.int32, device="cuda")
    nb = lib.conv_fprop_scratch_bytes(True, d)
    keep, sp = _scratch(torch, nb)
    for pr in (1, 0):
        lib.check(lib.raw().b2_conv_fprop_flex16(
            dI.data_ptr(), dF.data_ptr(), dO.data_ptr(), C.byref(d), table.data_ptr(), 0, 1, 2,
            stats.data_ptr(), sp, nb, probe.data_ptr(), status.data_ptr(), pr, 0))
        torch.cuda.synchronize()
        assert int(status.item()) == 0
    assert int(probe.item()) == int(np.abs(exact).max())
    if sh > 0:
        half = 1 << (sh - 1)
        exp = (exact + half - 1 + ((exact >> sh) & 1)) >> sh
    else:
        exp = exact
    exp = np.clip(exp, -32768, 32767)
    got = dO.cpu().numpy().astype(np.int64)
    assert np.array_equal(got, exp)
    assert int(stats[2].item()) == int(np.abs(got).max())


@pytest.mark.parametrize("flex", [0, 1])
def test_pool_avg(flex):
    import torch
    from ngraph_python_b200 import lib
    Cc, H, W, N = 64, 8, 8, 32
    rng = np.random.RandomState(5)
    if flex:
        x = rng.randint(-30000, 30000, (Cc, H, W, N)).astype(np.int16)
    else:
        x = rng.standard_normal((Cc, H, W, N)).astype(np.float32)
    dx = torch.from_numpy(x).cuda()
    out = torch.zeros((Cc, 1, 1, N), dtype=dx.dtype, device="cuda")
    stat = torch.zeros((1,), dtype=torch.int32, device="cuda")
    lib.check(lib.raw().b2_pool_avg_fprop(dx.data_ptr(), out.data_ptr(), flex, Cc, H, W, N, 1, 1,
                                          8, 8, 0, 0, 1, 1, stat.data_ptr(), 0))
    torch.cuda.synchronize()
    exp = co.pool_avg_fprop(x.astype(np.float32), (8, 8))
    if flex:
        assert np.abs(out.cpu().numpy().astype(np.float64) - exp).max() <= 0.5 + 1e-3
    else:
        np.testing.assert_allclose(out.cpu().numpy(), exp, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("flex", [0, 1])
def test_pool_max(flex):
    """Max pooling with padding and stride: exact in both storage types (the maximum of stored
    values; a flex16 result keeps the input's exponent)."""
    import torch
    from ngraph_python_b200 import lib
    Cc, H, W, N, R, S, pad, stride = 12, 9, 11, 32, 3, 3, 1, 2
    P, Q = (H + 2 * pad - R) // stride + 1, (W + 2 * pad - S) // stride + 1
    rng = np.random.RandomState(6)
    if flex:
        x = rng.randint(-30000, 30000, (Cc, H, W, N)).astype(np.int16)
    else:
        x = rng.standard_normal((Cc, H, W, N)).astype(np.float32)
    dx = torch.from_numpy(x).cuda()
    out = torch.zeros((Cc, P, Q, N), dtype=dx.dtype, device="cuda")
    stat = torch.zeros((1,), dtype=torch.int32, device="cuda")
    lib.check(lib.raw().b2_pool_max_fprop(dx.data_ptr(), out.data_ptr(), flex, Cc, H, W, N, P, Q,
                                          R, S, pad, pad, stride, stride, stat.data_ptr(), 0))
    torch.cuda.synchronize()
    exp = co.pool_max_fprop(x, (R, S), (pad, pad), (stride, stride))
    assert np.array_equal(out.cpu().numpy(), exp)
    if flex:
        assert int(stat.item()) == int(np.abs(exp.astype(np.int64)).max())


@pytest.mark.parametrize("op", ["avg", "max"])
@pytest.mark.parametrize("flex", [0, 1])
def test_pool_bprop(flex, op):
    """Gradient of pooling (overlapping windows, padding): fp32 equals the oracle's loop bit for
    bit (same order of additions); flex16 is the fp32 value quantised once."""
    import torch
    from ngraph_python_b200 import lib
    from oracle import flex_oracle as fx
    Cc, H, W, N, R, S, pad, stride = 6, 9, 11, 32, 3, 3, 1, 2
    P, Q = (H + 2 * pad - R) // stride + 1, (W + 2 * pad - S) // stride + 1
    rng = np.random.RandomState(8)
    if flex:
        xi = rng.randint(-30000, 30000, (Cc, H, W, N)).astype(np.int16)
        xi[:, 2:4, 3:6, :] = 777                      # ties: the first maximum must win
        ei = rng.randint(-30000, 30000, (Cc, P, Q, N)).astype(np.int16)
        dec_e = 12
        x, e = xi.astype(np.float32), ei.astype(np.float32) * np.float32(2.0 ** -dec_e)
    else:
        x = rng.standard_normal((Cc, H, W, N)).astype(np.float32)
        x[:, 2:4, 3:6, :] = 0.5
        e = rng.standard_normal((Cc, P, Q, N)).astype(np.float32)
        xi, ei = x, e
    exp = co.pool_bprop(e, x, (R, S), (pad, pad), (stride, stride), op)
    dx, de = torch.from_numpy(xi).cuda(), torch.from_numpy(ei).cuda()
    out = torch.zeros((Cc, H, W, N), dtype=dx.dtype, device="cuda")
    raw = lib.raw()
    if not flex:
        lib.check(raw.b2_pool_bprop(de.data_ptr(), dx.data_ptr(), out.data_ptr(), 0, int(op == "max"),
                                    Cc, H, W, N, P, Q, R, S, pad, pad, stride, stride, None, -1, -1,
                                    None, None, 0, 0))
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), exp)
        return
    dec_g = fx.fit_dec(float(np.abs(exp).max()))
    table = torch.tensor([[2.0 ** -dec_e, 2.0 ** dec_e], [2.0 ** -dec_g, 2.0 ** dec_g]],
                         dtype=torch.float32, device="cuda")
    stats = torch.zeros((2,), dtype=torch.int32, device="cuda")
    probe = torch.zeros((1,), dtype=torch.int64, device="cuda")
    for pr in (1, 0):
        lib.check(raw.b2_pool_bprop(de.data_ptr(), dx.data_ptr(), out.data_ptr(), 1, int(op == "max"),
                                    Cc, H, W, N, P, Q, R, S, pad, pad, stride, stride,
                                    table.data_ptr(), 0, 1, stats.data_ptr(), probe.data_ptr(), pr, 0))
    torch.cuda.synchronize()
    got_max = np.array([int(probe.item())], dtype=np.uint32).view(np.float32)[0]
    assert got_max == np.float32(np.abs(exp).max())
    want = fx.quantize(exp, dec_g).astype(np.int64)
    got = out.cpu().numpy().astype(np.int64)
    assert np.array_equal(got, want)
    assert int(stats[1].item()) == int(np.abs(got).max())


@pytest.mark.parametrize("axis", [0, 1])
@pytest.mark.parametrize("flex", [0, 1])
def test_lookup_table(flex, axis):
    """Embedding lookup and table gradient against oracle/lut_oracle.py: repeated indices, a
    padding index, indices never used.  fp32 with the table's rows looked up (axis 0): equal bit
    for bit (same order of additions)."""
    import torch
    from ngraph_python_b200 import lib
    from oracle import lut_oracle as lo
    from oracle import flex_oracle as fx
    V, F, n, pad_idx = 37, 24, 300, 5
    rng = np.random.RandomState(13 + axis)
    idx = rng.randint(0, V, n)
    idx[::9] = pad_idx
    idx[4::11] = idx[4]
    tshape = (V, F) if axis == 0 else (F, V)
    oshape = (n, F) if axis == 0 else (F, n)
    raw = lib.raw()
    if not flex:
        lut = rng.standard_normal(tshape).astype(np.float32)
        delta = rng.standard_normal(oshape).astype(np.float32)
        d_lut, d_idx, d_delta = [torch.from_numpy(a).cuda() for a in (lut, idx.astype(np.float32), delta)]
        out = torch.zeros(oshape, dtype=torch.float32, device="cuda")
        dW = torch.full(tshape, 7.0, dtype=torch.float32, device="cuda")
        lib.check(raw.b2_lut_fprop(d_lut.data_ptr(), d_idx.data_ptr(), out.data_ptr(), 0, axis, V, F,
                                   n, None, -1, 0))
        lib.check(raw.b2_lut_update(d_delta.data_ptr(), d_idx.data_ptr(), dW.data_ptr(), 0, axis, V,
                                    F, n, pad_idx, None, -1, -1, -1, None, None, 0, 0))
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), lo.lut_fprop(lut, idx, axis))
        want = lo.lut_update(delta, idx, pad_idx, axis, tshape)
        if axis == 0:
            assert np.array_equal(dW.cpu().numpy(), want)
        else:
            # along the contiguous axis numpy adds pairwise once a group has eight members; the
            # kernel adds in position order: same sums up to fp32 rounding
            np.testing.assert_allclose(dW.cpu().numpy(), want, rtol=2e-6, atol=2e-6)
        return
    lut = rng.randint(-30000, 30000, tshape).astype(np.int16)
    delta = rng.randint(-30000, 30000, oshape).astype(np.int16)
    dec_d, dec_i = 11, 0
    exp = lo.lut_update(delta.astype(np.float32) * np.float32(2.0 ** -dec_d), idx, pad_idx, axis, tshape)
    dec_w = fx.fit_dec(float(np.abs(exp).max()))
    d_lut, d_idx, d_delta = [torch.from_numpy(a).cuda() for a in (lut, idx.astype(np.int16), delta)]
    out = torch.zeros(oshape, dtype=torch.int16, device="cuda")
    dW = torch.full(tshape, 7, dtype=torch.int16, device="cuda")
    table = torch.tensor([[2.0 ** -d, 2.0 ** d] for d in (dec_d, dec_i, dec_w)], dtype=torch.float32,
                         device="cuda")
    stats = torch.zeros((3,), dtype=torch.int32, device="cuda")
    probe = torch.zeros((1,), dtype=torch.int64, device="cuda")
    lib.check(raw.b2_lut_fprop(d_lut.data_ptr(), d_idx.data_ptr(), out.data_ptr(), 1, axis, V, F, n,
                               table.data_ptr(), 1, 0))
    for pr in (1, 0):
        lib.check(raw.b2_lut_update(d_delta.data_ptr(), d_idx.data_ptr(), dW.data_ptr(), 1, axis, V, F,
                                    n, pad_idx, table.data_ptr(), 0, 1, 2, stats.data_ptr(),
                                    probe.data_ptr(), pr, 0))
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), lo.lut_fprop(lut, idx, axis))
    got_max = np.array([int(probe.item())], dtype=np.uint32).view(np.float32)[0]
    assert got_max == np.float32(np.abs(exp).max())
    want = fx.quantize(exp, dec_w).astype(np.int64)
    got = dW.cpu().numpy().astype(np.int64)
    assert np.array_equal(got, want)
    assert int(stats[2].item()) == int(np.abs(got).max())


# ---- the two training contractions ------------------------------------------------------------
# shapes of ResNet-20's layers (scaled down in H, W, N) plus ragged ones; the update contraction of
# the larger ones runs in several K slices
GRAD_SHAPES = [(16, 7, 7, 32, 8, 3, 3, 0, 1), (16, 9, 11, 32, 8, 3, 3, 1, 1), (3, 16, 16, 32, 16, 3, 3, 1, 1),
               (16, 16, 16, 64, 32, 3, 3, 1, 2), (32, 16, 16, 32, 64, 1, 1, 0, 2), (64, 8, 8, 32, 64, 3, 3, 1, 1),
               (5, 6, 5, 24, 10, 2, 3, 1, 1), (16, 12, 12, 256, 32, 3, 3, 1, 2), (16, 32, 32, 64, 16, 3, 3, 1, 1),
               (4, 9, 7, 10, 6, 3, 3, 1, 2),
               # unit stride and a batch that is a multiple of 128: the input gradient runs on the
               # implicit-GEMM kernel with flipped, transposed filters
               (16, 8, 8, 128, 16, 3, 3, 1, 1), (32, 6, 6, 128, 64, 3, 3, 1, 1),
               (16, 8, 8, 128, 32, 1, 1, 0, 1), (40, 5, 7, 128, 24, 3, 2, 1, 1),
               (64, 6, 6, 256, 130, 3, 3, 1, 1),
               # many k-blocks per slice of the filter-gradient kernel, two issuing threads
               (16, 32, 32, 256, 16, 3, 3, 1, 1), (3, 32, 32, 128, 16, 3, 3, 1, 1)]


def _run_grad(torch, lib, which, flex, first, second, out, d, table=None):
    status = torch.zeros((1,), dtype=torch.int32, device="cuda")
    sizer = lib.conv_bprop_scratch_bytes if which == "bprop" else lib.conv_update_scratch_bytes
    nb = sizer(bool(flex), d)
    keep, sp = _scratch(torch, nb)
    raw = lib.raw()
    if not flex:
        fn = raw.b2_conv_bprop_f32 if which == "bprop" else raw.b2_conv_update_f32
        lib.check(fn(first.data_ptr(), second.data_ptr(), out.data_ptr(), C.byref(d), sp, nb,
                     status.data_ptr(), 0))
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        return None
    fn = raw.b2_conv_bprop_flex16 if which == "bprop" else raw.b2_conv_update_flex16
    stats = torch.zeros((3,), dtype=torch.int32, device="cuda")
    probe = torch.zeros((1,), dtype=torch.int64, device="cuda")
    for pr in (1, 0):
        lib.check(fn(first.data_ptr(), second.data_ptr(), out.data_ptr(), C.byref(d),
                     table.data_ptr(), 0, 1, 2, stats.data_ptr(), sp, nb, probe.data_ptr(),
                     status.data_ptr(), pr, 0))
        torch.cuda.synchronize()
        assert int(status.item()) == 0
    return int(probe.item()), int(stats[2].item())


@pytest.mark.parametrize("which", ["bprop", "update"])
@pytest.mark.parametrize("shape", GRAD_SHAPES)
def test_conv_grad_f32(shape, which):
    import torch
    from ngraph_python_b200 import lib
    Cc, H, W, N, K, R, S, pad, stride = shape
    d, P, Q = _dims(lib, *shape)
    rng = np.random.RandomState(sum(shape) + 7)
    I = rng.standard_normal((Cc, H, W, N)).astype(np.float32)
    F = rng.standard_normal((Cc, R, S, K)).astype(np.float32)
    E = rng.standard_normal((K, P, Q, N)).astype(np.float32)
    dI, dF, dE = [torch.from_numpy(a).cuda() for a in (I, F, E)]
    if which == "bprop":
        out = torch.zeros((Cc, H, W, N), dtype=torch.float32, device="cuda")
        _run_grad(torch, lib, which, 0, dE, dF, out, d)
        exp = co.conv_bprop(E, F, (H, W), (pad, pad), (stride, stride), dtype=np.float64)
        terms = K * R * S
    else:
        out = torch.zeros((Cc, R, S, K), dtype=torch.float32, device="cuda")
        _run_grad(torch, lib, which, 0, dI, dE, out, d)
        exp = co.conv_update(I, E, (R, S), (pad, pad), (stride, stride), dtype=np.float64)
        terms = P * Q * N
    np.testing.assert_allclose(out.cpu().numpy(), exp, rtol=1e-4, atol=1e-5 * np.sqrt(terms) * 4)


@pytest.mark.parametrize("which", ["bprop", "update"])
@pytest.mark.parametrize("small", [True, False])
@pytest.mark.parametrize("shape", GRAD_SHAPES)
def test_conv_grad_flex16_exact(shape, small, which):
    import torch
    from ngraph_python_b200 import lib
    Cc, H, W, N, K, R, S, pad, stride = shape
    d, P, Q = _dims(lib, *shape)
    rng = np.random.RandomState(sum(shape) + 11)
    lim = 4 if small else 32767
    I = rng.randint(-lim, lim, (Cc, H, W, N)).astype(np.int16)
    F = rng.randint(-lim, lim, (Cc, R, S, K)).astype(np.int16)
    E = rng.randint(-lim, lim, (K, P, Q, N)).astype(np.int16)
    if which == "bprop":
        exact = co.conv_bprop(E, F, (H, W), (pad, pad), (stride, stride), dtype=np.int64)
        shape_o = (Cc, H, W, N)
    else:
        exact = co.conv_update(I, E, (R, S), (pad, pad), (stride, stride), dtype=np.int64)
        shape_o = (Cc, R, S, K)
    amax = int(np.abs(exact).max())
    sh = 0 if amax <= 32767 else int(np.ceil(np.log2(amax / 32767.0))) + 1
    table = torch.tensor([[1.0, 1.0], [1.0, 1.0], [2.0 ** sh, 2.0 ** -sh]], dtype=torch.float32,
                         device="cuda")
    dI, dF, dE = [torch.from_numpy(a).cuda() for a in (I, F, E)]
    out = torch.zeros(shape_o, dtype=torch.int16, device="cuda")
    if which == "bprop":
        probe, stat = _run_grad(torch, lib, which, 1, dE, dF, out, d, table)
    else:
        probe, stat = _run_grad(torch, lib, which, 1, dI, dE, out, d, table)
    assert probe == amax
    if sh > 0:
        half = 1 << (sh - 1)
        exp = (exact + half - 1 + ((exact >> sh) & 1)) >> sh
    else:
        exp = exact
    exp = np.clip(exp, -32768, 32767)
    got = out.cpu().numpy().astype(np.int64)
    assert np.array_equal(got, exp)
    assert stat == int(np.abs(got).max())


@pytest.mark.parametrize("variant", ["bias_relu", "bias_res_relu_planes", "bias_only"])
def test_conv_fused_epilogue(variant):
    """Bias / residual / ReLU folded into the tile kernel's epilogue, with the result also emitted
    as the byte planes the next convolution reads: one quantisation of the fp32 value."""
    import torch
    from ngraph_python_b200 import lib
    shape = (16, 8, 8, 128, 32, 3, 3, 1, 1)
    Cc, H, W, N, K, R, S, pad, stride = shape
    d, P, Q = _dims(lib, *shape)
    rng = np.random.RandomState(3)
    I = rng.randint(-20000, 20000, (Cc, H, W, N)).astype(np.int16)
    F = rng.randint(-20000, 20000, (Cc, R, S, K)).astype(np.int16)
    B = rng.randint(-20000, 20000, (K,)).astype(np.int16)
    Rz = rng.randint(-20000, 20000, (K, P, Q, N)).astype(np.int16)
    dec_i, dec_f, dec_b, dec_r = 12, 15, 13, 10
    exact = co.conv_fprop(I, F, (pad, pad), (stride, stride), dtype=np.int64)
    y = exact.astype(np.float64) * 2.0 ** -(dec_i + dec_f)
    y = y.astype(np.float32) + B.astype(np.float32)[:, None, None, None] * np.float32(2.0 ** -dec_b)
    use_res = variant == "bias_res_relu_planes"
    if use_res:
        y = y + Rz.astype(np.float32) * np.float32(2.0 ** -dec_r)
    if variant != "bias_only":
        y = np.maximum(y, 0)
    from oracle import flex_oracle as fx
    dec_o = fx.fit_dec(float(np.abs(y).max()))
    exp = fx.quantize(y, dec_o).astype(np.int64)
    ok, act_bytes, filt_bytes = lib.conv_planes_info(d, lib.CONV_FPROP)
    assert ok
    dI, dF, dB, dR = [torch.from_numpy(a).cuda() for a in (I, F, B, Rz)]
    keep_a, act = _scratch(torch, 2 * act_bytes)
    keep_f, filt = _scratch(torch, filt_bytes)
    out = torch.zeros((K, P, Q, N), dtype=torch.int16, device="cuda")
    out_plane_bytes = (K * P * Q * N + 1023) // 1024 * 1024
    keep_o, oplanes = _scratch(torch, 2 * out_plane_bytes)
    table = torch.tensor([[2.0 ** -dd, 2.0 ** dd] for dd in (dec_i, dec_f, dec_o, dec_b, dec_r)],
                         dtype=torch.float32, device="cuda")
    stats = torch.zeros((5,), dtype=torch.int32, device="cuda")
    probe = torch.zeros((1,), dtype=torch.int64, device="cuda")
    status = torch.zeros((1,), dtype=torch.int32, device="cuda")
    raw = lib.raw()
    lib.check(raw.b2_conv_split_activations(dI.data_ptr(), C.byref(d), 0, act, 0))
    lib.check(raw.b2_conv_filter_planes(dF.data_ptr(), C.byref(d), 0, filt, 0))
    epi = lib.ConvEpilogue()
    epi.bias, epi.slot_bias = dB.data_ptr(), 3
    epi.residual, epi.slot_residual = (dR.data_ptr(), 4) if use_res else (None, -1)
    epi.relu = int(variant != "bias_only")
    epi.write_int16 = 1
    epi.out_planes, epi.plane_bytes = (oplanes, out_plane_bytes) if use_res else (None, 0)
    for pr in (1, 0):
        lib.check(raw.b2_conv_flex16_planes_fused(0, act, filt, out.data_ptr(), C.byref(d),
                                                  table.data_ptr(), 0, 1, 2, C.byref(epi),
                                                  stats.data_ptr(), probe.data_ptr(),
                                                  status.data_ptr(), pr, 0))
        torch.cuda.synchronize()
        assert int(status.item()) == 0
    got_max = np.array([int(probe.item())], dtype=np.uint32).view(np.float32)[0]
    assert abs(got_max - float(np.abs(y).max())) <= 1e-5 * float(np.abs(y).max())
    got = out.cpu().numpy().astype(np.int64)
    # the integer sum is converted to fp32 once (the oracle above goes through float64): one step
    assert np.abs(got - exp).max() <= 1
    assert (got != exp).mean() < 0.01
    assert int(stats[2].item()) == int(np.abs(got).max())
    if use_res:
        pl = keep_o.cpu().numpy()
        off = oplanes - keep_o.data_ptr()
        hi = pl[off:off + got.size].view(np.int8).astype(np.int64).reshape(got.shape)
        lo = pl[off + out_plane_bytes:off + out_plane_bytes + got.size].astype(np.int64).reshape(got.shape)
        assert np.array_equal(256 * hi + lo, got)


# ---- the reference's own flex convolution shape set, with its depth axes ------------------------
# tests/flex_tests/test_flexconv.py:25-45: (H, W, D, R, S, T, (pad_h, pad_w, pad_d),
# (str_h, str_w, str_d)); C = 16, N = 32, K = 8, integer data in [-4, 4), exact equality (:60-70).
REF_FLEXCONV = [
    (7, 7, 1, 3, 3, 1, (0, 0, 0), (1, 1, 1)), (5, 5, 1, 3, 3, 1, (1, 1, 1), (1, 1, 1)),
    (10, 10, 1, 4, 4, 1, (3, 3, 3), (1, 1, 1)), (7, 7, 2, 3, 3, 2, (0, 0, 0), (1, 1, 1)),
    (8, 8, 1, 4, 4, 1, (0, 0, 0), (2, 2, 2)), (10, 10, 1, 3, 3, 1, (1, 1, 1), (3, 3, 3)),
    (7, 7, 1, 3, 3, 1, (1, 2, 3), (1, 1, 1)), (7, 7, 1, 3, 3, 1, (0, 3, 0), (1, 1, 1)),
    (7, 7, 1, 3, 3, 1, (0, 0, 0), (3, 1, 1)), (7, 7, 1, 3, 3, 1, (0, 0, 0), (1, 2, 3)),
]
# its three "limitation" cases (:47-52: K not a multiple of 8, N not a multiple of 32, dilation)
# are assertion failures of the reference's SASS kernels; here they are ordinary supported shapes
# (H, W, D, R, S, T, pad, stride, K, N, dilation)
REF_FLEXCONV_LIMITS = [(7, 7, 1, 3, 3, 1, (0, 0, 0), (1, 1, 1), 7, 32, 1),
                       (7, 7, 1, 3, 3, 1, (0, 0, 0), (1, 1, 1), 8, 31, 1),
                       (7, 7, 1, 3, 3, 1, (0, 0, 0), (1, 1, 1), 8, 32, 2),
                       (9, 8, 3, 3, 2, 2, (2, 1, 1), (2, 1, 1), 12, 40, 2)]


def _dims3(lib, Cc, N, K, H, W, D, R, S, T, pad, stride, dil=1):
    ph, pw, pd = pad
    sh, sw, sd = stride
    d = lib.ConvDims()
    d.C, d.D, d.H, d.W, d.N = Cc, D, H, W, N
    d.K, d.T, d.R, d.S = K, T, R, S
    d.M = (D + 2 * pd - dil * (T - 1) - 1) // sd + 1
    d.P = (H + 2 * ph - dil * (R - 1) - 1) // sh + 1
    d.Q = (W + 2 * pw - dil * (S - 1) - 1) // sw + 1
    d.pad_d, d.pad_h, d.pad_w = pd, ph, pw
    d.str_d, d.str_h, d.str_w = sd, sh, sw
    d.dil_d = d.dil_h = d.dil_w = dil
    return d


def _flexconv_cases():
    out = [(16, 32, 8) + s + (1,) for s in REF_FLEXCONV]
    for (H, W, D, R, S, T, pad, stride, K, N, dil) in REF_FLEXCONV_LIMITS:
        out.append((16, N, K, H, W, D, R, S, T, pad, stride, dil))
    return out


@pytest.mark.parametrize("flex", [True, False])
@pytest.mark.parametrize("case", _flexconv_cases())
def test_reference_flexconv_shapes_all_three_contractions(case, flex):
    """Forward, input gradient and filter gradient on every shape of the reference's flex
    convolution test (depth 2, 4x4 filters with padding 3, stride 3, asymmetric padding and
    stride) and on its three limitation cases, through the C ABI: flex16 results are the exact
    integer contractions (np.array_equal, as the reference asserts), fp32 within rtol 1e-4."""
    import torch
    from ngraph_python_b200 import lib
    Cc, N, K, H, W, D, R, S, T, pad, stride, dil = case
    d = _dims3(lib, Cc, N, K, H, W, D, R, S, T, pad, stride, dil)
    rng = np.random.RandomState(abs(hash(case)) % (2 ** 31))
    I = rng.randint(-4, 4, (Cc, D, H, W, N))
    F = rng.randint(-4, 4, (Cc, T, R, S, K))
    E = rng.randint(-4, 4, (K, d.M, d.P, d.Q, N))
    p3, s3, d3 = (pad[2], pad[0], pad[1]), (stride[2], stride[0], stride[1]), (dil, dil, dil)
    want = [co.conv3d_fprop(I, F, p3, s3, d3, np.int64),
            co.conv3d_bprop(E, F, (D, H, W), p3, s3, d3, np.int64),
            co.conv3d_update(I, E, (T, R, S), p3, s3, d3, np.int64)]
    raw = lib.raw()
    dt_np, dt_t = (np.int16, torch.int16) if flex else (np.float32, torch.float32)
    dI, dF, dE = [torch.from_numpy(x.astype(dt_np)).cuda() for x in (I, F, E)]
    status = torch.zeros((1,), dtype=torch.int32, device="cuda")
    table = torch.ones((3, 2), dtype=torch.float32, device="cuda")      # all exponents 0
    stats = torch.zeros((3,), dtype=torch.int32, device="cuda")
    probe = torch.zeros((1,), dtype=torch.int64, device="cuda")
    jobs = [("fprop", lib.conv_fprop_scratch_bytes, raw.b2_conv_fprop_flex16, raw.b2_conv_fprop_f32,
             (dI, dF)),
            ("bprop", lib.conv_bprop_scratch_bytes, raw.b2_conv_bprop_flex16, raw.b2_conv_bprop_f32,
             (dE, dF)),
            ("update", lib.conv_update_scratch_bytes, raw.b2_conv_update_flex16,
             raw.b2_conv_update_f32, (dI, dE))]
    for (name, sizer, f16, f32, (a, b)), exp in zip(jobs, want):
        out = torch.zeros(exp.shape, dtype=dt_t, device="cuda")
        nb = sizer(flex, d)
        keep, sp = _scratch(torch, nb)
        if flex:
            assert int(np.abs(exp).max()) <= 32767
            stats.zero_()
            probe.zero_()
            for pr in (1, 0):
                lib.check(f16(a.data_ptr(), b.data_ptr(), out.data_ptr(), C.byref(d),
                              table.data_ptr(), 0, 1, 2, stats.data_ptr(), sp, nb, probe.data_ptr(),
                              status.data_ptr(), pr, 0))
                torch.cuda.synchronize()
                assert int(status.item()) == 0
            assert int(probe.item()) == int(np.abs(exp).max()), name
            assert np.array_equal(out.cpu().numpy().astype(np.int64), exp), name
            assert int(stats[2].item()) == int(np.abs(exp).max()), name
        else:
            lib.check(f32(a.data_ptr(), b.data_ptr(), out.data_ptr(), C.byref(d), sp, nb,
                          status.data_ptr(), 0))
            torch.cuda.synchronize()
            assert int(status.item()) == 0
            np.testing.assert_allclose(out.cpu().numpy(), exp, rtol=1e-4, atol=1e-3, err_msg=name)


@pytest.mark.parametrize("flex", [True, False])
@pytest.mark.parametrize("case", _flexconv_cases())
def test_reference_flexconv_shapes_through_the_transformer(case, flex):
    """The same set the way the reference runs it (ngraph/testing/flex_util.py:241-267,
    execute_convolution): placeholders for image and filters, ng.convolution, one call of the
    computation with integer data; the result must equal the numpy convolution exactly."""
    import ngraph_python_b200 as ng
    Cc, N, K, H, W, D, R, S, T, pad, stride, dil = case
    ax = lambda n, nm: ng.make_axis(n, name=nm)   # noqa: E731
    M = (D + 2 * pad[2] - dil * (T - 1) - 1) // stride[2] + 1
    P = (H + 2 * pad[0] - dil * (R - 1) - 1) // stride[0] + 1
    Q = (W + 2 * pad[1] - dil * (S - 1) - 1) // stride[1] + 1
    ax_i = [ax(Cc, "C"), ax(D, "D"), ax(H, "H"), ax(W, "W"), ax(N, "N")]
    ax_f = [ax_i[0], ax(T, "T"), ax(R, "R"), ax(S, "S"), ax(K, "K")]
    ax_o = [ax_f[4], ax(M, "M"), ax(P, "P"), ax(Q, "Q"), ax_i[4]]
    params = dict(pad_d=pad[2], pad_h=pad[0], pad_w=pad[1], str_d=stride[2], str_h=stride[0],
                  str_w=stride[1], dil_d=dil, dil_h=dil, dil_w=dil)
    rng = np.random.RandomState(3)
    iv = rng.randint(-4, 4, [a.length for a in ax_i]).astype(np.float32)
    fv = rng.randint(-4, 4, [a.length for a in ax_f]).astype(np.float32)
    t = ng.transformers.allocate_transformer("b200", flex=flex)
    inputs, filters = ng.placeholder(ax_i), ng.placeholder(ax_f)
    comp = t.computation(ng.convolution(params, inputs, filters, axes=ax_o), inputs, filters)
    got = comp(iv, fv)
    t.close()
    exp = co.conv3d_fprop(iv, fv, (pad[2], pad[0], pad[1]), (stride[2], stride[0], stride[1]),
                          (dil, dil, dil), np.float64)
    assert np.array_equal(np.asarray(got, dtype=np.float64), exp)
