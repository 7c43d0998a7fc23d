"""CPU restatement of the library's random fill (ngraph_python_b200/csrc/b2_rng.cu).

TEST INFRASTRUCTURE ONLY.  The reference fills random tensors through pycuda's generator
(ngraph/transformers/gpu/tensor_ops.py:621-661) and its CPU transformer through numpy's; neither
stream can be reproduced by the other, and the reference's own test only checks ranges and
moments (tests/transformer_dependent/test_rngop.py).  What CAN be pinned bit for bit is this
library's generator against the published algorithm it names: Philox-4x32 with 10 rounds (Salmon,
Moraes, Dror, Shaw, SC'11), restated here with numpy integers, with the known-answer vectors of
that paper's reference implementation checked in tests/test_rng_oracle.py.
"""
import numpy as np

M0, M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
W0, W1 = 0x9E3779B9, 0xBB67AE85
MASK = np.uint64(0xFFFFFFFF)


def philox4x32_10(counters, key):
    """counters: (n, 4) uint32; key: (k0, k1) -> (n, 4) uint32."""
    c = [counters[:, i].astype(np.uint64) for i in range(4)]
    k0, k1 = int(key[0]) & 0xFFFFFFFF, int(key[1]) & 0xFFFFFFFF
    for _ in range(10):
        p0 = M0 * c[0]
        p1 = M1 * c[2]
        hi0, lo0 = p0 >> np.uint64(32), p0 & MASK
        hi1, lo1 = p1 >> np.uint64(32), p1 & MASK
        c = [hi1 ^ c[1] ^ np.uint64(k0), lo1, hi0 ^ c[3] ^ np.uint64(k1), lo0]
        k0 = (k0 + W0) & 0xFFFFFFFF
        k1 = (k1 + W1) & 0xFFFFFFFF
    return np.stack([x.astype(np.uint32) for x in c], axis=1)


def words(n, seed, offset):
    """The 32-bit words the fill uses for elements 0..n-1: group g = i // 4 has the counter
    (g_lo, g_hi, offset_lo, offset_hi) under the key (seed_lo, seed_hi)."""
    groups = (n + 3) // 4
    g = np.arange(groups, dtype=np.uint64)
    ctr = np.stack([(g & MASK), (g >> np.uint64(32)),
                    np.full(groups, offset & 0xFFFFFFFF, np.uint64),
                    np.full(groups, (offset >> 32) & 0xFFFFFFFF, np.uint64)], axis=1).astype(np.uint32)
    return philox4x32_10(ctr, (seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)).reshape(-1)[:4 * groups]


def u01(w):
    return (w >> np.uint32(8)).astype(np.float32) * np.float32(1.0 / 16777216.0)


def uniform(n, low, high, seed, offset):
    """fp32, operation for operation as the kernel: low + (high - low) * u, folded back to low
    where rounding lands on high."""
    lo, hi = np.float32(low), np.float32(high)
    x = lo + (hi - lo) * u01(words(n, seed, offset))
    x = np.where((x < hi) | ~(lo < hi), x, lo).astype(np.float32)
    return x[:n]


def normal(n, loc, scale, seed, offset):
    """Box-Muller on word pairs (w0, w1) and (w2, w3) of every group; float64 here, so the kernel
    (fp32 logf / sincospif) agrees to a few ulp, not bit for bit."""
    w = words(n, seed, offset).reshape(-1, 2)
    r = np.sqrt(-2.0 * np.log(1.0 - u01(w[:, 0]).astype(np.float64)))
    ang = 2.0 * np.pi * u01(w[:, 1]).astype(np.float64)
    out = np.stack([r * np.cos(ang), r * np.sin(ang)], axis=1).reshape(-1)
    return (loc + scale * out)[:n]
