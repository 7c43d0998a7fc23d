"""The numpy restatement of Philox-4x32-10 (oracle/rng_oracle.py) against the known-answer vectors
published with the algorithm's reference implementation (counter, key -> output), and the basic
properties of the derived uniform / normal streams."""
import numpy as np

from oracle import rng_oracle as ro

KAT = [((0, 0, 0, 0), (0, 0), (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)),
       ((0xffffffff,) * 4, (0xffffffff, 0xffffffff),
        (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)),
       ((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0),
        (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1))]


def test_philox_known_answers():
    for ctr, key, want in KAT:
        got = ro.philox4x32_10(np.array([ctr], dtype=np.uint32), key)[0]
        assert tuple(int(x) for x in got) == want


def test_streams():
    u = ro.uniform(100003, -0.5, 0.5, seed=7, offset=3)
    assert u.dtype == np.float32 and u.shape == (100003,)
    assert u.min() >= -0.5 and u.max() < 0.5 and abs(float(u.mean())) < 5e-3
    assert np.array_equal(u, ro.uniform(100003, -0.5, 0.5, seed=7, offset=3))
    assert not np.array_equal(u, ro.uniform(100003, -0.5, 0.5, seed=7, offset=4))
    assert np.array_equal(u[:1000], ro.uniform(1000, -0.5, 0.5, seed=7, offset=3))
    g = ro.normal(200000, -0.5, 2.0, seed=1, offset=0)
    assert abs(g.mean() + 0.5) < 0.02 and abs(g.std() - 2.0) < 0.02
