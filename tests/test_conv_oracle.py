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
