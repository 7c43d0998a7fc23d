"""GPU parity of the tcgen05 GEMM kernels through the C ABI.

flex16: the exact integer product sum is computed by the oracle in int64; the kernel's mantissas
must be within +-1 of round(sum * 2^(decC-decA-decB)) (the bar for flex contractions), and are in
fact expected to be identical because both sides are exact.  fp32: rtol 1e-4 / atol 1e-5 scaled
by sqrt(K) against a float64 product."""
import numpy as np
import pytest

from oracle import flex_oracle as fx

pytestmark = pytest.mark.gpu


def _scratch(torch, nbytes):
    t = torch.empty((nbytes + 1024,), dtype=torch.uint8, device="cuda")
    off = (-t.data_ptr()) % 1024
    return t, t.data_ptr() + off


SHAPES = [(128, 128, 128), (256, 384, 512), (100, 72, 200), (1, 10, 64), (512, 128, 1024),
          (130, 257, 96),
          # K above 32768: the flex16 contraction runs in slices of exact int32 sums
          (64, 48, 40000)]


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("layout", ["nn", "nt", "tn"])
def test_gemm_f32(M, N, K, layout):
    import torch
    from ngraph_python_b200 import lib
    rng = np.random.RandomState(M + N + K)
    A = rng.standard_normal((M, K)).astype(np.float32)
    B = rng.standard_normal((K, N)).astype(np.float32)
    a_store = A.T.copy() if layout == "tn" else A
    b_store = B.T.copy() if layout == "nt" else B
    a_str = (1, M) if layout == "tn" else (K, 1)
    b_str = (1, K) if layout == "nt" else (N, 1)
    dA, dB = torch.from_numpy(a_store).cuda(), torch.from_numpy(b_store).cuda()
    dC = torch.zeros((M, N), dtype=torch.float32, device="cuda")
    status = torch.zeros((1,), dtype=torch.int32, device="cuda")
    nbytes = lib.gemm_scratch_bytes(False, M, N, K)
    keep, sp = _scratch(torch, nbytes)
    lib.check(lib.raw().b2_gemm_f32(dA.data_ptr(), a_str[0], a_str[1], dB.data_ptr(), b_str[0],
                                    b_str[1], dC.data_ptr(), N, M, N, K, sp, nbytes,
                                    status.data_ptr(), 0))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    expect = A.astype(np.float64) @ B.astype(np.float64)
    np.testing.assert_allclose(dC.cpu().numpy(), expect, rtol=1e-4, atol=1e-5 * np.sqrt(K) * 4)


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("layout", ["nn", "nt", "tn"])
def test_gemm_flex16(M, N, K, layout):
    import torch
    from ngraph_python_b200 import lib
    rng = np.random.RandomState(M * 3 + N + K)
    A = rng.randint(-32767, 32768, (M, K)).astype(np.int16)
    B = rng.randint(-32767, 32768, (K, N)).astype(np.int16)
    A[0, 0] = -32768
    B[0, 0] = -32768
    dec_a, dec_b = 15, 12
    exact = A.astype(np.int64) @ B.astype(np.int64)
    real_max = float(np.abs(exact).max()) * 2.0 ** -(dec_a + dec_b)
    dec_c = fx.fit_dec(real_max)
    a_store = A.T.copy() if layout == "tn" else A
    b_store = B.T.copy() if layout == "nt" else B
    a_str = (1, M) if layout == "tn" else (K, 1)
    b_str = (1, K) if layout == "nt" else (N, 1)
    dA, dB = torch.from_numpy(a_store).cuda(), torch.from_numpy(b_store).cuda()
    dC = torch.zeros((M, N), dtype=torch.int16, device="cuda")
    table = torch.tensor([[2.0 ** -dec_a, 2.0 ** dec_a], [2.0 ** -dec_b, 2.0 ** dec_b],
                          [2.0 ** -dec_c, 2.0 ** dec_c]], dtype=torch.float32, device="cuda")
    stats = torch.zeros((3,), dtype=torch.int32, device="cuda")
    probe = torch.zeros((1,), dtype=torch.int64, device="cuda")
    status = torch.zeros((1,), dtype=torch.int32, device="cuda")
    nbytes = lib.gemm_scratch_bytes(True, M, N, K)
    keep, sp = _scratch(torch, nbytes)

    def call(probe_flag):
        lib.check(lib.raw().b2_gemm_flex16(
            dA.data_ptr(), a_str[0], a_str[1], dB.data_ptr(), b_str[0], b_str[1], dC.data_ptr(), N,
            M, N, K, table.data_ptr(), 0, 1, 2, stats.data_ptr(), sp, nbytes, probe.data_ptr(),
            status.data_ptr(), probe_flag, 0))
        torch.cuda.synchronize()
        assert int(status.item()) == 0
    call(1)
    assert int(probe.item()) == int(np.abs(exact).max())
    call(0)
    sh = dec_a + dec_b - dec_c
    # round-to-nearest-even of exact / 2^sh in exact integer arithmetic
    if sh > 0:
        half = 1 << (sh - 1)
        expect = (exact + half - 1 + ((exact >> sh) & 1)) >> sh
    else:
        expect = exact << (-sh)
    expect = np.clip(expect, -32768, 32767)
    got = dC.cpu().numpy().astype(np.int64)
    assert np.array_equal(got, expect)
    assert int(stats[2].item()) == int(np.abs(got).max())
    # and with a deliberately too-fine output exponent everything saturates cleanly
    table[2, 0] = 2.0 ** -(dec_c + 6)
    table[2, 1] = 2.0 ** (dec_c + 6)
    stats.zero_()
    call(0)
    sh2 = sh - 6
    if sh2 > 0:
        half = 1 << (sh2 - 1)
        e2 = (exact + half - 1 + ((exact >> sh2) & 1)) >> sh2
    else:
        e2 = exact << (-sh2)
    e2 = np.clip(e2, -32768, 32767)
    assert np.array_equal(dC.cpu().numpy().astype(np.int64), e2)


# ---- benchmark configuration 3 at its stated sizes ---------------------------------------------
# int16 products summed over K <= 8192 stay below 2^45: a float64 BLAS product is an exact oracle.
def _rne_shift(exact, sh):
    if sh > 0:
        half = 1 << (sh - 1)
        out = (exact + half - 1 + ((exact >> sh) & 1)) >> sh
    else:
        out = exact << (-sh)
    return np.clip(out, -32768, 32767)


def _stored(X, transposed):
    return np.ascontiguousarray(X.T) if transposed else X


@pytest.mark.parametrize("n", [1024, 4096, 8192])
def test_gemm_flex16_benchmark_sizes(n):
    """M = N = K = n, mantissas uniform in [-32767, 32767], exponents -15 and -12 (benchmark
    configuration 3), all three operand layouts, the output exponent chosen from the probe launch as the
    transformer chooses it; then once more with an exponent six bits too fine, where most of
    the output saturates.  1024 and 4096 are checked in full, 8192 on 48 sampled rows."""
    import torch
    from ngraph_python_b200 import lib
    rng = np.random.RandomState(n)
    A = rng.randint(-32767, 32768, (n, n)).astype(np.int16)
    B = rng.randint(-32767, 32768, (n, n)).astype(np.int16)
    rows = np.arange(n) if n <= 4096 else np.sort(rng.choice(n, 48, replace=False))
    exact = np.rint(A[rows].astype(np.float64) @ B.astype(np.float64)).astype(np.int64)
    dec_a, dec_b = 15, 12
    nbytes = lib.gemm_scratch_bytes(True, n, n, n)
    keep, sp = _scratch(torch, nbytes)
    stats = torch.zeros((3,), dtype=torch.int32, device="cuda")
    probe = torch.zeros((1,), dtype=torch.int64, device="cuda")
    status = torch.zeros((1,), dtype=torch.int32, device="cuda")
    dC = torch.zeros((n, n), dtype=torch.int16, device="cuda")
    for layout in ("nn", "nt", "tn"):
        dA = torch.from_numpy(_stored(A, layout == "tn")).cuda()
        dB = torch.from_numpy(_stored(B, layout == "nt")).cuda()
        a_str = (1, n) if layout == "tn" else (n, 1)
        b_str = (1, n) if layout == "nt" else (n, 1)
        table = torch.zeros((3, 2), dtype=torch.float32, device="cuda")
        table[0, 0], table[0, 1] = 2.0 ** -dec_a, 2.0 ** dec_a
        table[1, 0], table[1, 1] = 2.0 ** -dec_b, 2.0 ** dec_b

        def call(probe_flag):
            lib.check(lib.raw().b2_gemm_flex16(
                dA.data_ptr(), a_str[0], a_str[1], dB.data_ptr(), b_str[0], b_str[1],
                dC.data_ptr(), n, n, n, n, table.data_ptr(), 0, 1, 2, stats.data_ptr(), sp, nbytes,
                probe.data_ptr(), status.data_ptr(), probe_flag, 0))
            torch.cuda.synchronize()
            assert int(status.item()) == 0
        probe.zero_()
        call(1)
        imax = int(probe.item())
        if n <= 4096:
            assert imax == int(np.abs(exact).max())
        else:
            assert imax >= int(np.abs(exact).max())
        dec_c = fx.fit_dec(float(imax) * 2.0 ** -(dec_a + dec_b))
        for extra in (0, 6):
            d = dec_c + extra
            table[2, 0], table[2, 1] = 2.0 ** -d, 2.0 ** d
            stats.zero_()
            call(0)
            got = dC[torch.from_numpy(rows).cuda()].cpu().numpy().astype(np.int64)
            expect = _rne_shift(exact, dec_a + dec_b - d)
            assert np.array_equal(got, expect), (layout, extra)
            if extra:
                assert (np.abs(expect) >= 32767).mean() > 0.5      # it does saturate
                assert int(stats[2].item()) == 32768 or int(stats[2].item()) == 32767
            elif n <= 4096:
                assert int(stats[2].item()) == int(np.abs(got).max())
        del dA, dB


@pytest.mark.parametrize("n", [1024, 4096, 8192])
def test_gemm_f32_benchmark_sizes(n):
    """The fp32 twin of benchmark configuration 3: A, B ~ N(0,1), all three layouts, against a
    float64 product at rtol 1e-4 / atol 1e-5 * 4 sqrt(K) (a sum of K products of unit variance
    has magnitude sqrt(K)).  8192 is checked on 48 sampled rows."""
    import torch
    from ngraph_python_b200 import lib
    rng = np.random.RandomState(n + 1)
    A = rng.standard_normal((n, n)).astype(np.float32)
    B = rng.standard_normal((n, n)).astype(np.float32)
    rows = np.arange(n) if n <= 4096 else np.sort(rng.choice(n, 48, replace=False))
    expect = A[rows].astype(np.float64) @ B.astype(np.float64)
    nbytes = lib.gemm_scratch_bytes(False, n, n, n)
    keep, sp = _scratch(torch, nbytes)
    status = torch.zeros((1,), dtype=torch.int32, device="cuda")
    dC = torch.zeros((n, n), dtype=torch.float32, device="cuda")
    for layout in ("nn", "nt", "tn"):
        dA = torch.from_numpy(_stored(A, layout == "tn")).cuda()
        dB = torch.from_numpy(_stored(B, layout == "nt")).cuda()
        a_str = (1, n) if layout == "tn" else (n, 1)
        b_str = (1, n) if layout == "nt" else (n, 1)
        dC.zero_()
        lib.check(lib.raw().b2_gemm_f32(dA.data_ptr(), a_str[0], a_str[1], dB.data_ptr(), b_str[0],
                                        b_str[1], dC.data_ptr(), n, n, n, n, sp, nbytes,
                                        status.data_ptr(), 0))
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        got = dC[torch.from_numpy(rows).cuda()].cpu().numpy()
        np.testing.assert_allclose(got, expect, rtol=1e-4, atol=1e-5 * np.sqrt(n) * 4,
                                   err_msg=layout)
        del dA, dB


def test_bounded_wait_runs_out_and_reports():
    """A device-side wait that nothing completes gives up after its poll limit, sets the status
    word and lets the kernel end normally (tensor memory freed): the library's self-test runs that
    path with the tile kernels' own wait routine on a barrier nobody arrives at.  Afterwards the
    context is as usable as before -- a GEMM on the same stream is exact -- and a transformer
    turns a non-zero status word into an error for that call, then clears it."""
    import torch
    import ngraph_python_b200 as ng
    from ngraph_python_b200 import lib
    status = torch.zeros((1,), dtype=torch.int32, device="cuda")
    waited = torch.zeros((1,), dtype=torch.int32, device="cuda")
    lib.check(lib.raw().b2_selftest_bounded_wait(300, status.data_ptr(), waited.data_ptr(), 0))
    torch.cuda.synchronize()
    assert int(status.item()) == 1 and int(waited.item()) == 300
    with pytest.raises(lib.B200Error, match="poll limit"):
        lib.check(lib.raw().b2_selftest_bounded_wait(0, status.data_ptr(), None, 0))
    # the tensor cores and tensor memory are as before
    M_, K_, N_ = [ng.make_axis(n, name=nm) for n, nm in ((128, "M"), (256, "K"), (128, "N"))]
    a, b = ng.placeholder([M_, K_]), ng.placeholder([K_, N_])
    t = ng.transformers.allocate_transformer("b200")
    comp = t.computation(ng.dot(a, b), a, b)
    rng = np.random.RandomState(1)
    av = rng.randint(-8, 8, (128, 256)).astype(np.float32)
    bv = rng.randint(-8, 8, (256, 128)).astype(np.float32)
    assert np.array_equal(comp(av, bv), av @ bv)
    # what a computation does when one of its kernels reports a wait that ran out
    lib.check(lib.raw().b2_selftest_bounded_wait(50, t._status.data_ptr(), None,
                                                 t.stream.cuda_stream))
    with pytest.raises(lib.B200Error, match="device-side wait ran out"):
        comp(av, bv)
    assert np.array_equal(comp(av, bv), av @ bv)       # the word was cleared; the next call is fine
    t.close()
