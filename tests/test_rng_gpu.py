"""Random fill on the device: the generator bit for bit against its numpy restatement
(oracle/rng_oracle.py, itself pinned to the published known-answer vectors), and the behaviour the
reference's own test asks of ng.uniform / ng.normal (tests/transformer_dependent/test_rngop.py:
ranges, moments, fresh numbers on every execution)."""
import numpy as np
import pytest

from oracle import rng_oracle as ro

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [1, 5, 4096, 100003])
def test_uniform_bit_exact_and_normal_close(n):
    import torch
    from ngraph_python_b200 import lib
    raw = lib.raw()
    out = torch.zeros((n,), dtype=torch.float32, device="cuda")
    seed, offset = 0x1234567887654321, (3 << 40) + 17
    lib.check(raw.b2_rng_fill(out.data_ptr(), 0, n, lib.RNG_UNIFORM, -0.25, 0.75, seed, offset, None,
                              None, -1, None, None, 0, 0))
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), ro.uniform(n, -0.25, 0.75, seed, offset))
    lib.check(raw.b2_rng_fill(out.data_ptr(), 0, n, lib.RNG_NORMAL, -0.5, 2.0, seed, offset, None,
                              None, -1, None, None, 0, 0))
    torch.cuda.synchronize()
    np.testing.assert_allclose(out.cpu().numpy(), ro.normal(n, -0.5, 2.0, seed, offset),
                               rtol=2e-5, atol=2e-5)
    # a device counter is added to the offset and advanced by the storing launch
    ctr = torch.tensor([5], dtype=torch.int64, device="cuda")
    lib.check(raw.b2_rng_fill(out.data_ptr(), 0, n, lib.RNG_UNIFORM, 0.0, 1.0, seed, offset,
                              ctr.data_ptr(), None, -1, None, None, 0, 0))
    torch.cuda.synchronize()
    assert int(ctr.item()) == 6
    assert np.array_equal(out.cpu().numpy(), ro.uniform(n, 0.0, 1.0, seed, offset + 5))


def test_flex16_fill_quantises_the_same_numbers():
    import torch
    from oracle import flex_oracle as fx
    from ngraph_python_b200 import lib
    n, dec = 50000, 13
    out = torch.zeros((n,), dtype=torch.int16, device="cuda")
    table = torch.tensor([[2.0 ** -dec, 2.0 ** dec]], dtype=torch.float32, device="cuda")
    stats = torch.zeros((1,), dtype=torch.int32, device="cuda")
    probe = torch.zeros((1,), dtype=torch.int64, device="cuda")
    args = (out.data_ptr(), 1, n, lib.RNG_UNIFORM, -2.0, 3.0, 9, 1, None, table.data_ptr(), 0,
            stats.data_ptr(), probe.data_ptr())
    lib.check(lib.raw().b2_rng_fill(*(args + (1, 0))))
    lib.check(lib.raw().b2_rng_fill(*(args + (0, 0))))
    torch.cuda.synchronize()
    want = ro.uniform(n, -2.0, 3.0, 9, 1)
    bits = np.array([int(probe.item()) & 0xffffffff], dtype=np.uint32).view(np.float32)[0]
    assert bits == np.abs(want).max()
    q = fx.quantize(want, dec)
    assert np.array_equal(out.cpu().numpy(), q)
    assert int(stats[0].item()) == fx.maxabs_stat(q)


@pytest.mark.parametrize("flex", [False, True])
def test_rng_ops_through_the_transformer(flex):
    import ngraph_python_b200 as ng
    M, N = ng.make_axis(100, name="M"), ng.make_axis(100, name="N")
    base = ng.persistent_tensor([M, N], initial_value=10.0)
    t = ng.transformers.allocate_transformer("b200", flex=flex, rng_seed=3)
    uni = t.computation(ng.uniform(base, low=-0.5, high=0.5))
    nrm = t.computation(ng.normal(base, loc=-0.5, scale=1.0))
    both = t.computation(ng.sum(ng.uniform(base), reduction_axes=[M, N]))
    u = np.array(uni(), copy=True)
    assert u.shape == (100, 100)
    assert np.all(u < 0.5) and np.all(u >= -0.5) and not np.all(u >= 0.0)
    g = np.array(nrm(), copy=True)
    assert np.allclose(np.mean(g), -0.5, rtol=0.1, atol=0.02)
    assert np.allclose(np.std(g), 1.0, rtol=0.1, atol=0.02)
    # every execution draws again (test_rng_repetition), also when replayed from a CUDA graph
    v1, v2 = float(both()), float(both())
    assert v1 != v2
    both.capture()
    v3, v4 = float(both()), float(both())
    assert len({v1, v2, v3, v4}) == 4
    u2 = np.array(uni(), copy=True)
    assert not np.array_equal(u, u2)
    t.close()
    # the seed fixes the streams
    t2 = ng.transformers.allocate_transformer("b200", flex=flex, rng_seed=3)
    base2 = ng.persistent_tensor([M, N], initial_value=10.0)
    uni2 = t2.computation(ng.uniform(base2, low=-0.5, high=0.5))
    assert np.array_equal(np.array(uni2()), u)
    t2.close()
