"""GPU parity of the fused elementwise/reduction kernels, called through the C ABI, against the
numpy oracle on the same seeded inputs."""
import numpy as np
import pytest

from oracle import ew_oracle as ew
from oracle import flex_oracle as fx

pytestmark = pytest.mark.gpu


def _torch():
    import torch
    return torch


def c2_program(lib, rows, cols, flex):
    """y = tanh(a*x+b)*sigmoid(c); s = sum(y, axis 1); m = max(|y|, axis 1)."""
    dt = lib.FLEX16 if flex else lib.F32
    ins = [dict(dtype=dt, slot=i if flex else -1, strides=(0, cols, 1)) for i in range(4)]
    ops = [("mul", 1, 0), ("add", 4, 2), ("tanh", 5, None), ("sig", 3, None), ("mul", 6, 7),
           ("abs", 8, None)]
    outs = [dict(dtype=dt, slot=4 if flex else -1, strides=(0, cols, 1), reg=8)]
    reds = [dict(dtype=dt, slot=5 if flex else -1, strides=(0, 1, 0), reg=8, redop="sum"),
            dict(dtype=dt, slot=6 if flex else -1, strides=(0, 1, 0), reg=9, redop="max")]
    return lib.make_program((1, rows, cols), ins, [], ops, outs, reds, lib.REDUCE_C)


def c2_oracle(x, a, b, c):
    t = ew.apply("add", ew.apply("mul", a, x), b)
    y = ew.apply("mul", ew.apply("tanh", t), ew.apply("sig", c))
    return y, y.astype(np.float64).sum(axis=1), np.abs(y).max(axis=1)


@pytest.mark.parametrize("rows,cols", [(64, 4096), (7, 1000), (5, 333), (300, 40), (2, 1 << 20)])
def test_c2_fp32(rows, cols):
    torch = _torch()
    from ngraph_python_b200 import lib
    rng = np.random.RandomState(0)
    host = [rng.standard_normal((rows, cols)).astype(np.float32) for _ in range(4)]
    dev = [torch.from_numpy(h).cuda() for h in host]
    y = torch.empty((rows, cols), dtype=torch.float32, device="cuda")
    s = torch.empty((rows,), dtype=torch.float32, device="cuda")
    m = torch.empty((rows,), dtype=torch.float32, device="cuda")
    k = lib.EwKernel(c2_program(lib, rows, cols, False))
    scratch = torch.empty((max(k.scratch_bytes, 4),), dtype=torch.uint8, device="cuda")
    k.launch([d.data_ptr() for d in dev], [y.data_ptr(), s.data_ptr(), m.data_ptr()],
             scratch=scratch.data_ptr(), scratch_bytes=k.scratch_bytes)
    torch.cuda.synchronize()
    ey, es, em = c2_oracle(*host)
    # fp32 bar: rtol 1e-4 / atol 1e-5
    np.testing.assert_allclose(y.cpu().numpy(), ey, rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(s.cpu().numpy(), es, rtol=1e-4, atol=1e-5 * cols)
    np.testing.assert_allclose(m.cpu().numpy(), em, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("rows,cols", [(64, 4096), (7, 1000), (5, 333), (2, 1 << 20)])
def test_c2_flex16(rows, cols):
    torch = _torch()
    from ngraph_python_b200 import lib
    rng = np.random.RandomState(1)
    host = [rng.standard_normal((rows, cols)).astype(np.float32) for _ in range(4)]
    decs = [fx.fit_dec(float(np.abs(h).max())) for h in host]
    mants = [fx.host_to_mantissa(h, d)[0] for h, d in zip(host, decs)]
    vals = [fx.dequantize(mm, d) for mm, d in zip(mants, decs)]
    ey, es, em = c2_oracle(*vals)
    out_decs = [fx.fit_dec(float(np.abs(ey).max())), fx.fit_dec(float(np.abs(es).max())),
                fx.fit_dec(float(np.abs(em).max()))]
    table = np.zeros((7, 2), dtype=np.float32)
    for i, d in enumerate(decs + out_decs):
        table[i] = (2.0 ** -d, 2.0 ** d)
    d_table = torch.from_numpy(table).cuda()
    d_stats = torch.zeros((7,), dtype=torch.int32, device="cuda")
    dev = [torch.from_numpy(mm).cuda() for mm in mants]
    y = torch.empty((rows, cols), dtype=torch.int16, device="cuda")
    s = torch.empty((rows,), dtype=torch.int16, device="cuda")
    m = torch.empty((rows,), dtype=torch.int16, device="cuda")
    k = lib.EwKernel(c2_program(lib, rows, cols, True))
    scratch = torch.empty((max(k.scratch_bytes, 4),), dtype=torch.uint8, device="cuda")
    outs = [y.data_ptr(), s.data_ptr(), m.data_ptr()]
    # probe pass: the unsaturated fp32 range of each output, as float bit patterns
    k.launch([d.data_ptr() for d in dev], outs, flex_table=d_table.data_ptr(),
             flex_stats=d_stats.data_ptr(), scratch=scratch.data_ptr(),
             scratch_bytes=k.scratch_bytes, probe=True)
    torch.cuda.synchronize()
    probe = d_stats.cpu().numpy()[4:7].view(np.float32)
    np.testing.assert_allclose(probe[0], np.abs(ey).max(), rtol=1e-5)
    np.testing.assert_allclose(probe[1], np.abs(es).max(), rtol=1e-4)
    np.testing.assert_allclose(probe[2], np.abs(em).max(), rtol=1e-5)
    d_stats.zero_()
    k.launch([d.data_ptr() for d in dev], outs, flex_table=d_table.data_ptr(),
             flex_stats=d_stats.data_ptr(), scratch=scratch.data_ptr(),
             scratch_bytes=k.scratch_bytes)
    torch.cuda.synchronize()
    gy = y.cpu().numpy()
    qy = fx.quantize(ey, out_decs[0])
    # tanh/exp come from two different libms: the quantised mantissa may differ by one unit
    # where the fp32 value sits on a rounding boundary; everything else is bit-exact.
    diff = np.abs(gy.astype(np.int32) - qy.astype(np.int32))
    assert diff.max() <= 1
    assert (diff != 0).mean() < 2e-3
    assert int(d_stats[4].item()) == fx.maxabs_stat(gy)
    gm = m.cpu().numpy()
    dm = np.abs(gm.astype(np.int32) - fx.quantize(em, out_decs[2]).astype(np.int32))
    assert dm.max() <= 1
    assert int(d_stats[6].item()) == fx.maxabs_stat(gm)
    gs = s.cpu().numpy().astype(np.float64) * 2.0 ** -out_decs[1]
    np.testing.assert_allclose(gs, es, rtol=1e-3, atol=8 * 2.0 ** -out_decs[1] + 1e-4 * cols ** 0.5)


def test_arith_flex_bit_exact():
    """add/sub/mul/div/max/min are IEEE-exact: the flex result must match the oracle bit for bit,
    including saturation and the statistic."""
    torch = _torch()
    from ngraph_python_b200 import lib
    rng = np.random.RandomState(2)
    n = 1 << 16
    xa = (rng.standard_normal(n) * 3).astype(np.float32)
    xb = (rng.standard_normal(n) * 0.5).astype(np.float32)
    da, db = fx.fit_dec(np.abs(xa).max()), fx.fit_dec(np.abs(xb).max())
    ma, mb = fx.host_to_mantissa(xa, da)[0], fx.host_to_mantissa(xb, db)[0]
    va, vb = fx.dequantize(ma, da), fx.dequantize(mb, db)
    for name in ("add", "sub", "mul", "div", "maximum", "minimum"):
        expect = ew.apply(name, va, vb)
        out_dec = 10  # deliberately too fine for some values: exercises saturation
        table = np.array([[2.0 ** -da, 2.0 ** da], [2.0 ** -db, 2.0 ** db],
                          [2.0 ** -out_dec, 2.0 ** out_dec]], dtype=np.float32)
        d_table = torch.from_numpy(table).cuda()
        d_stats = torch.zeros((3,), dtype=torch.int32, device="cuda")
        ins = [dict(dtype=lib.FLEX16, slot=0, strides=(0, 0, 1)),
               dict(dtype=lib.FLEX16, slot=1, strides=(0, 0, 1))]
        outs = [dict(dtype=lib.FLEX16, slot=2, strides=(0, 0, 1), reg=2)]
        k = lib.EwKernel(lib.make_program((1, 1, n), ins, [], [(name, 0, 1)], outs, [],
                                          lib.REDUCE_NONE))
        a, b = torch.from_numpy(ma).cuda(), torch.from_numpy(mb).cuda()
        y = torch.empty((n,), dtype=torch.int16, device="cuda")
        k.launch([a.data_ptr(), b.data_ptr()], [y.data_ptr()], flex_table=d_table.data_ptr(),
                 flex_stats=d_stats.data_ptr())
        torch.cuda.synchronize()
        q = fx.quantize(expect, out_dec)
        assert np.array_equal(y.cpu().numpy(), q), name
        assert int(d_stats[2].item()) == fx.maxabs_stat(q), name


def test_host_quantize_roundtrip():
    torch = _torch()
    from ngraph_python_b200 import lib
    rng = np.random.RandomState(3)
    x = (rng.standard_normal(100003) * 7).astype(np.float32)
    x[5] = 1e9
    x[6] = -1e9
    dec = 11
    table = torch.tensor([[2.0 ** -dec, 2.0 ** dec]], dtype=torch.float32, device="cuda")
    stats = torch.zeros((1,), dtype=torch.int32, device="cuda")
    src = torch.from_numpy(x).cuda()
    dst = torch.empty((x.size,), dtype=torch.int16, device="cuda")
    lib.check(lib.raw().b2_flex_host_quantize(src.data_ptr(), dst.data_ptr(), x.size,
                                              table.data_ptr(), 0, stats.data_ptr(), 0))
    torch.cuda.synchronize()
    em, emax = fx.host_to_mantissa(x, dec)
    assert np.array_equal(dst.cpu().numpy(), em)
    assert int(stats[0].item()) == emax
    back = torch.empty((x.size,), dtype=torch.float32, device="cuda")
    lib.check(lib.raw().b2_flex_dequantize(dst.data_ptr(), back.data_ptr(), x.size,
                                           table.data_ptr(), 0, 0))
    torch.cuda.synchronize()
    assert np.array_equal(back.cpu().numpy(), fx.dequantize(em, dec))
    bits = torch.zeros((1,), dtype=torch.int32, device="cuda")
    lib.check(lib.raw().b2_absmax_bits_f32(src.data_ptr(), x.size, bits.data_ptr(), 0))
    assert bits.cpu().numpy().view(np.float32)[0] == np.abs(x).max()


@pytest.mark.parametrize("flex", [False, True])
def test_c2_at_benchmark_size_on_sampled_rows(flex):
    """Benchmark configuration 2 at its stated size, 8192 x 16384: the kernel runs over the whole
    tensor, 64 sampled rows (the first, the last, and rows on either side of every 1024-row
    boundary among them) are checked against the oracle with the bars of the small cases.
    Inputs are drawn on the device; the flex16 run quantises them there with the library's own
    host-write kernel, and the oracle gets the mantissas of the sampled rows."""
    torch = _torch()
    from ngraph_python_b200 import lib
    rows, cols = 8192, 16384
    gen = torch.Generator(device="cuda")
    gen.manual_seed(7)
    dev32 = [torch.randn((rows, cols), device="cuda", generator=gen) for _ in range(4)]
    rs = np.random.RandomState(5)
    pick = sorted(set([0, rows - 1] + [b + d for b in range(1024, rows, 1024) for d in (-1, 0)] +
                      list(rs.choice(rows, 48, replace=False))))[:64]
    idx = torch.tensor(pick, device="cuda")
    k = lib.EwKernel(c2_program(lib, rows, cols, flex))
    scratch = torch.empty((max(k.scratch_bytes, 4),), dtype=torch.uint8, device="cuda")
    dt = torch.int16 if flex else torch.float32
    y = torch.empty((rows, cols), dtype=dt, device="cuda")
    s = torch.empty((rows,), dtype=dt, device="cuda")
    m = torch.empty((rows,), dtype=dt, device="cuda")
    outs = [y.data_ptr(), s.data_ptr(), m.data_ptr()]
    if not flex:
        k.launch([d.data_ptr() for d in dev32], outs, scratch=scratch.data_ptr(),
                 scratch_bytes=k.scratch_bytes)
        torch.cuda.synchronize()
        host = [d[idx].cpu().numpy() for d in dev32]
        ey, es, em = c2_oracle(*host)
        np.testing.assert_allclose(y[idx].cpu().numpy(), ey, rtol=1e-4, atol=1e-5)
        np.testing.assert_allclose(s[idx].cpu().numpy(), es, rtol=1e-4, atol=1e-5 * cols)
        np.testing.assert_allclose(m[idx].cpu().numpy(), em, rtol=1e-4, atol=1e-5)
        return
    decs = [fx.fit_dec(float(d.abs().max().item())) for d in dev32]
    out_decs = [14, 6, 14]          # |y| < 1; |row sum| stays far below 512; row max|y| < 1
    table = np.zeros((7, 2), dtype=np.float32)
    for i, d in enumerate(decs + out_decs):
        table[i] = (2.0 ** -d, 2.0 ** d)
    d_table = torch.from_numpy(table).cuda()
    d_stats = torch.zeros((7,), dtype=torch.int32, device="cuda")
    dev = []
    for i, d32 in enumerate(dev32):
        q = torch.empty((rows, cols), dtype=torch.int16, device="cuda")
        lib.check(lib.raw().b2_flex_host_quantize(d32.data_ptr(), q.data_ptr(), rows * cols,
                                                  d_table.data_ptr(), i, d_stats.data_ptr(), 0))
        dev.append(q)
    torch.cuda.synchronize()
    # the device conversion is the oracle's host write, on the sampled rows
    for i in range(4):
        assert np.array_equal(dev[i][idx].cpu().numpy(),
                              fx.host_to_mantissa(dev32[i][idx].cpu().numpy(), decs[i])[0])
    del dev32
    d_stats.zero_()
    k.launch([d.data_ptr() for d in dev], outs, flex_table=d_table.data_ptr(),
             flex_stats=d_stats.data_ptr(), scratch=scratch.data_ptr(),
             scratch_bytes=k.scratch_bytes)
    torch.cuda.synchronize()
    vals = [fx.dequantize(d[idx].cpu().numpy(), dec) for d, dec in zip(dev, decs)]
    ey, es, em = c2_oracle(*vals)
    gy = y[idx].cpu().numpy()
    diff = np.abs(gy.astype(np.int32) - fx.quantize(ey, out_decs[0]).astype(np.int32))
    assert diff.max() <= 1 and (diff != 0).mean() < 2e-3
    gm = m[idx].cpu().numpy()
    assert np.abs(gm.astype(np.int32) - fx.quantize(em, out_decs[2]).astype(np.int32)).max() <= 1
    gs = s[idx].cpu().numpy().astype(np.float64) * 2.0 ** -out_decs[1]
    np.testing.assert_allclose(gs, es, rtol=1e-3, atol=8 * 2.0 ** -out_decs[1] + 1e-4 * cols ** 0.5)
    # the statistic covers the whole tensor: it is the maximum over everything that was stored
    assert int(d_stats[4].item()) == int(y.to(torch.int32).abs().max().item())
    assert int(d_stats[6].item()) == int(m.to(torch.int32).abs().max().item())
