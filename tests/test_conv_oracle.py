"""The numpy convolution/pooling restatement against outputs of the reference's CPU transformer
(fixtures) -- pins the oracle that the GPU kernel tests and the CPU baseline use."""
import os

import numpy as np
import pytest

import ngraph_python_b200 as ng
from oracle import conv_oracle as co
from tests.golden import cases

FIX = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "fixtures")


def _check(name, pad, stride):
    _, _, vals = cases.CASES[name](ng)
    I, F = vals
    got = co.conv_fprop(I[:, 0], F[:, 0], (pad, pad), (stride, stride))
    exp = np.load(os.path.join(FIX, name + ".npz"))["out0_0"][:, 0]
    np.testing.assert_allclose(got, exp, rtol=1e-4, atol=1e-4)


def test_conv_oracle_matches_reference_cpu():
    _check("conv_basic", 1, 1)
    _check("conv_stride2_1x1", 0, 2)
    _check("conv_stride2_3x3", 1, 2)


def test_pool_oracle():
    x = np.arange(2 * 4 * 4 * 3, dtype=np.float32).reshape(2, 4, 4, 3)
    out = co.pool_avg_fprop(x, (4, 4))
    np.testing.assert_allclose(out[:, 0, 0, :], x.reshape(2, 16, 3).mean(axis=1))
    out = co.pool_avg_fprop(x, (2, 2), stride=(2, 2))
    np.testing.assert_allclose(out[1, 1, 0, 2], x[1, 2:4, 0:2, 2].mean())
    out = co.pool_max_fprop(x, (3, 3), pad=(1, 1), stride=(2, 2))
    assert out.shape == (2, 2, 2, 3)
    assert out[1, 0, 0, 2] == x[1, 0:2, 0:2, 2].max()          # window clipped by the padding
    assert out[0, 1, 1, 1] == x[0, 1:4, 1:4, 1].max()


@pytest.mark.parametrize("shape", [(3, 7, 6, 4, 5, 3, 3, 1, 1), (4, 9, 8, 2, 6, 3, 2, 1, 2),
                                   (2, 8, 8, 3, 4, 1, 1, 0, 2), (5, 6, 6, 2, 3, 2, 2, 0, 1)])
def test_gradient_oracles_are_the_adjoints_of_fprop(shape):
    """<fprop(I, F), E> = <I, bprop(E, F)> = <F, update(I, E)> holds exactly in integers: the
    gradient restatements are the transposes of the forward restatement, which the reference
    fixtures pin."""
    Cc, H, W, N, K, R, S, pad, stride = shape
    rng = np.random.RandomState(sum(shape))
    I = rng.randint(-9, 10, (Cc, H, W, N)).astype(np.int64)
    F = rng.randint(-9, 10, (Cc, R, S, K)).astype(np.int64)
    O = co.conv_fprop(I, F, (pad, pad), (stride, stride), dtype=np.int64)
    E = rng.randint(-9, 10, O.shape).astype(np.int64)
    gI = co.conv_bprop(E, F, (H, W), (pad, pad), (stride, stride), dtype=np.int64)
    U = co.conv_update(I, E, (R, S), (pad, pad), (stride, stride), dtype=np.int64)
    assert gI.shape == I.shape and U.shape == F.shape
    lhs = int((O * E).sum())
    assert lhs == int((I * gI).sum())
    assert lhs == int((F * U).sum())


@pytest.mark.parametrize("shape", [(5, 9, 11, 3, 6, 3, 3, 1, 2), (4, 8, 8, 2, 7, 1, 1, 0, 2),
                                   (3, 10, 7, 2, 5, 3, 2, 1, 2), (6, 7, 7, 2, 4, 3, 3, 1, 1),
                                   (3, 12, 9, 2, 4, 3, 3, 0, 2), (2, 9, 9, 2, 3, 2, 2, 0, 1)])
def test_input_gradient_is_a_unit_stride_convolution_of_the_dilated_error(shape):
    """The identity the tile kernel uses for input gradients, on exact integers: put zeros
    between the elements of E (a tensor H+2pad-R+1 high, E at the multiples of the stride), flip
    and transpose the filters, pad by R-1-pad, convolve with unit stride."""
    C, H, W, N, K, R, S, pad, stride = shape
    P = (H + 2 * pad - R) // stride + 1
    Q = (W + 2 * pad - S) // stride + 1
    rng = np.random.RandomState(sum(shape))
    E = rng.randint(-300, 300, (K, P, Q, N)).astype(np.int64)
    F = rng.randint(-300, 300, (C, R, S, K)).astype(np.int64)
    want = co.conv_bprop(E, F, (H, W), (pad, pad), (stride, stride), dtype=np.int64)
    he, we = H + 2 * pad - R + 1, W + 2 * pad - S + 1
    assert he >= (P - 1) * stride + 1 and we >= (Q - 1) * stride + 1
    dil = np.zeros((K, he, we, N), np.int64)
    dil[:, :(P - 1) * stride + 1:stride, :(Q - 1) * stride + 1:stride, :] = E
    flipped = np.ascontiguousarray(F[:, ::-1, ::-1, :].transpose(3, 1, 2, 0))      # (K, R, S, C)
    got = co.conv_fprop(dil, flipped, (R - 1 - pad, S - 1 - pad), (1, 1), dtype=np.int64)
    assert got.shape == want.shape
    assert np.array_equal(got, want)


def test_folding_the_output_step_into_the_epilogue_is_exact():
    """The fused convolution epilogue multiplies every term by the output's 1/step (a power of
    two) instead of scaling the finished fp32 value: same bits, as long as nothing overflows or
    goes subnormal."""
    rng = np.random.RandomState(5)
    acc = rng.randint(-2 ** 38, 2 ** 38, 20000).astype(np.float64).astype(np.float32)
    bias = (rng.randint(-32768, 32768, 20000) * 2.0 ** -13).astype(np.float32)
    res = (rng.randint(-32768, 32768, 20000) * 2.0 ** -10).astype(np.float32)
    for dec_in, dec_out in ((27, 11), (20, 3), (30, 14), (12, -2)):
        f = np.float32(2.0 ** -dec_in)
        q = np.float32(2.0 ** dec_out)
        plain = ((res + (acc * f + bias).astype(np.float32)).astype(np.float32) * q).astype(np.float32)
        folded = (res * q + (acc * (f * q) + bias * q).astype(np.float32)).astype(np.float32)
        assert np.array_equal(plain, folded)


@pytest.mark.parametrize("op", ["avg", "max"])
def test_pool_gradient_oracle_is_the_adjoint(op):
    """<pool(I + t d), E> differentiated at t = 0 equals <d, pool_bprop(E)> (max: away from
    ties, where the pooling is differentiable)."""
    rng = np.random.RandomState(4)
    I = rng.standard_normal((3, 7, 8, 4)).astype(np.float64)
    E = rng.standard_normal((3, 4, 4, 4)).astype(np.float64)
    d = rng.standard_normal(I.shape)
    ana = (co.pool_bprop(E.astype(np.float32), I.astype(np.float32), (3, 3), (1, 1), (2, 2), op)
           .astype(np.float64) * d).sum()
    if op == "avg":                     # linear: <pool(d), E> itself
        num = (co.pool_avg_fprop(d.astype(np.float32), (3, 3), (1, 1), (2, 2)).astype(np.float64) * E).sum()
    else:
        eps = 1e-6
        num = ((co.pool_max_fprop(I + eps * d, (3, 3), (1, 1), (2, 2)) -
                co.pool_max_fprop(I - eps * d, (3, 3), (1, 1), (2, 2))) * E).sum() / (2 * eps)
    assert abs(num - ana) <= 2e-3 * max(1.0, abs(ana))


def test_depth_oracles_match_reference_cpu():
    """The restatements with depth axes, asymmetric padding / stride and dilation against the
    reference CPU transformer's forward result and both gradients (fixture conv3d_grads), and,
    with D = T = M = 1, against the 2-d restatements."""
    _, _, (I, F, E) = cases.CASES["conv3d_grads"](ng)
    fix = np.load(os.path.join(FIX, "conv3d_grads.npz"))
    geo = ((1, 2, 0), (1, 2, 1), (1, 1, 2))
    np.testing.assert_allclose(co.conv3d_fprop(I, F, *geo), fix["out0_0"], rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(co.conv3d_bprop(E, F, I.shape[1:4], *geo), fix["out0_1"], rtol=1e-4,
                               atol=1e-4)
    np.testing.assert_allclose(co.conv3d_update(I, E, F.shape[1:4], *geo), fix["out0_2"], rtol=1e-4,
                               atol=2e-3)
    rng = np.random.RandomState(3)
    I2 = rng.randint(-9, 10, (4, 9, 8, 2)).astype(np.int64)
    F2 = rng.randint(-9, 10, (4, 3, 2, 6)).astype(np.int64)
    O2 = co.conv_fprop(I2, F2, (1, 1), (2, 1), dtype=np.int64)
    assert np.array_equal(co.conv3d_fprop(I2[:, None], F2[:, None], (0, 1, 1), (1, 2, 1),
                                          dtype=np.int64)[:, 0], O2)
    E2 = rng.randint(-9, 10, O2.shape).astype(np.int64)
    assert np.array_equal(co.conv3d_bprop(E2[:, None], F2[:, None], (1, 9, 8), (0, 1, 1), (1, 2, 1),
                                          dtype=np.int64)[:, 0],
                          co.conv_bprop(E2, F2, (9, 8), (1, 1), (2, 1), dtype=np.int64))
    assert np.array_equal(co.conv3d_update(I2[:, None], E2[:, None], (1, 3, 2), (0, 1, 1), (1, 2, 1),
                                           dtype=np.int64)[:, 0],
                          co.conv_update(I2, E2, (3, 2), (1, 1), (2, 1), dtype=np.int64))
