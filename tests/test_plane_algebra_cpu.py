"""The integer algebra behind the flex16 tensor-core kernels, restated in numpy and checked
against plain int64 products: an int16 mantissa m = 256*hi + lo (hi signed, lo unsigned byte), the
second operand's low plane stored as the signed byte lo - 128 so that both of its planes are one
signed int8 operand, and the correction 128 * (sum of the first operand) that this costs."""
import numpy as np
import pytest


def split(m):
    m = m.astype(np.int64)
    lo = m & 0xff
    return (m - lo) >> 8, lo            # hi in [-128, 127], lo in [0, 255]


@pytest.mark.parametrize("K", [32, 160, 4096])
def test_merged_operand_form(K):
    """GEMM and convolution forward / input gradient: A_hi x [B_hi | B_lo'] and A_lo x [B_hi |
    B_lo'] accumulate HH | X and X | LL; v = HH*65536 + X*256 + LL + 128*rowsum(A)."""
    rng = np.random.RandomState(K)
    A = rng.randint(-32768, 32768, (24, K))
    B = rng.randint(-32768, 32768, (K, 20))
    ah, al = split(A)
    bh, bl = split(B)
    blp = bl - 128
    assert blp.min() >= -128 and blp.max() <= 127
    HH = ah @ bh
    X = ah @ blp + al @ bh
    LL = al @ blp
    rowsum = A.astype(np.int64).sum(axis=1, keepdims=True)
    v = HH * 65536 + X * 256 + LL + 128 * rowsum
    assert np.array_equal(v, A.astype(np.int64) @ B.astype(np.int64))
    # the convolution kernel takes the row sums from one more column of B that is (0, +1):
    # its X entry is sum(A_hi), its LL entry sum(A_lo)
    s_hi, s_lo = ah.sum(axis=1, keepdims=True), al.sum(axis=1, keepdims=True)
    assert np.array_equal(256 * s_hi + s_lo, rowsum)
    # int32 accumulators: every partial sum stays below 2^31 up to 32768 terms
    assert 2 * 128 * 255 * 32768 < 2 ** 31


def test_filter_gradient_form():
    """Filter gradient: accumulators [HH | Ah*El'] and [Al*Eh | LL] kept apart (each starts from
    zero), two issuing threads with sets of their own, row sums from a constant row of B."""
    rng = np.random.RandomState(3)
    A = rng.randint(-32768, 32768, (126, 1024))          # rows (c,r,s), contraction over images
    E = rng.randint(-32768, 32768, (17, 1024))           # rows k
    ah, al = split(A)
    eh, el = split(E)
    elp = el - 128
    total = np.zeros((126, 17), np.int64)
    fix = np.zeros((126, 1), np.int64)
    for issuer in range(2):                               # alternate 128-image blocks
        cols = np.concatenate([np.arange(b, b + 128) for b in range(issuer * 128, 1024, 256)])
        hh = ah[:, cols] @ eh[:, cols].T
        x1 = ah[:, cols] @ elp[:, cols].T
        x2 = al[:, cols] @ eh[:, cols].T
        ll = al[:, cols] @ elp[:, cols].T
        ones_hi, ones_lo = 0, 1                          # the constant row: (hi, lo') = (0, +1)
        s_hi = ah[:, cols].sum(axis=1, keepdims=True) * ones_lo + 0 * ones_hi
        s_lo = al[:, cols].sum(axis=1, keepdims=True) * ones_lo
        total += hh * 65536 + (x1 + x2) * 256 + ll
        fix += 128 * (256 * s_hi + s_lo)
    assert np.array_equal(total + fix, A.astype(np.int64) @ E.astype(np.int64).T)


def test_requant_is_what_store_and_load_give():
    """B2_OP_REQUANT: round-to-nearest-even of v / step, saturated to int16, times the step --
    and storing that value again reproduces the same mantissa (the op is idempotent)."""
    rng = np.random.RandomState(9)
    v = (rng.standard_normal(50000) * 3).astype(np.float32)
    for dec in (8, 12, 15):
        q, s = np.float32(2.0 ** dec), np.float32(2.0 ** -dec)
        m = np.clip(np.rint(v * q), -32768, 32767).astype(np.int32)
        back = m.astype(np.float32) * s
        m2 = np.clip(np.rint(back * q), -32768, 32767).astype(np.int32)
        assert np.array_equal(m, m2)
