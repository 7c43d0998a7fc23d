"""The numpy convolution/pooling restatement against outputs of the reference's CPU transformer
(fixtures) -- pins the oracle that the GPU kernel tests and the CPU baseline use."""
import os

import numpy as np

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
