"""N-d strided copy / transpose (b2_dimshuffle) through the C ABI and through the transformer,
against numpy.  Bit-exact: the kernel moves elements, it does not compute.

Shapes follow what the reference exercises (tests/transformer_dependent/test_dimshuffle.py: a 2-d
transpose; test_dimshuffle_op.py: 3-d to 5-d reorders feeding convolutions and dots) plus ragged
extents, every element size, sliced views and ranks up to the limit of 8."""
import itertools

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _strides(shape):
    out, acc = [], 1
    for n in reversed(shape):
        out.append(acc)
        acc *= n
    return list(reversed(out))


CASES = [((2, 3), (1, 0)), ((129, 257), (1, 0)), ((64, 48, 40), (2, 0, 1)), ((33, 7, 65), (1, 2, 0)),
         ((16, 1, 12, 10, 32), (4, 0, 1, 2, 3)), ((8, 3, 3, 16), (3, 1, 2, 0)),
         ((5, 4, 3, 6, 2, 7), (5, 3, 1, 0, 2, 4)), ((2, 3, 2, 3, 2, 3, 2, 3), (7, 6, 5, 4, 3, 2, 1, 0)),
         ((1000,), (0,)), ((4, 5, 6), (0, 1, 2)), ((1, 1, 1), (2, 1, 0))]


@pytest.mark.parametrize("esize", [1, 2, 4, 8])
@pytest.mark.parametrize("shape,perm", CASES)
def test_dimshuffle_c_abi(shape, perm, esize):
    """dst (dense, axes in `perm` order) <- src (dense): numpy's transpose."""
    import torch
    from ngraph_python_b200 import lib
    dt = {1: np.uint8, 2: np.int16, 4: np.float32, 8: np.int64}[esize]
    rng = np.random.RandomState(sum(shape) + esize)
    x = rng.randint(0, 120, shape).astype(dt)
    want = np.ascontiguousarray(np.transpose(x, perm))
    src = torch.from_numpy(x).cuda()
    dst = torch.zeros(want.shape, dtype=src.dtype, device="cuda")
    # iterate in the SOURCE's axis order: destination strides are those of the permuted tensor
    dstr_perm = _strides(want.shape)
    dst_strides = [0] * len(shape)
    for pos, a in enumerate(perm):
        dst_strides[a] = dstr_perm[pos]
    lib.dimshuffle(src.data_ptr(), dst.data_ptr(), esize, list(shape), _strides(shape), dst_strides)
    torch.cuda.synchronize()
    assert np.array_equal(dst.cpu().numpy(), want)


def test_dimshuffle_c_abi_sliced_views_and_broadcast():
    import torch
    from ngraph_python_b200 import lib
    rng = np.random.RandomState(1)
    x = rng.standard_normal((20, 30, 40)).astype(np.float32)
    # a strided window of the source, written transposed into a window of a larger destination
    win = x[2:18:2, 5:25, 1:40:3]                       # (8, 20, 13)
    out = np.full((13, 25, 8), -7.0, np.float32)
    src, dst = torch.from_numpy(x).cuda(), torch.from_numpy(out).cuda()
    s = _strides(x.shape)
    d = _strides(out.shape)
    lib.dimshuffle(src.data_ptr() + 4 * (2 * s[0] + 5 * s[1] + 1), dst.data_ptr() + 4 * (3 * d[1]),
                   4, [8, 20, 13], [2 * s[0], s[1], 3 * s[2]], [d[2], d[1], d[0]])
    torch.cuda.synchronize()
    out[:, 3:23, :] = np.transpose(win, (2, 1, 0))
    assert np.array_equal(dst.cpu().numpy(), out)
    # a source stride of 0 broadcasts
    row = rng.standard_normal(50).astype(np.float32)
    srow = torch.from_numpy(row).cuda()
    full = torch.zeros((7, 50), dtype=torch.float32, device="cuda")
    lib.dimshuffle(srow.data_ptr(), full.data_ptr(), 4, [7, 50], [0, 1], [50, 1])
    torch.cuda.synchronize()
    assert np.array_equal(full.cpu().numpy(), np.broadcast_to(row, (7, 50)))
    with pytest.raises(lib.B200Error, match="rank"):
        lib.dimshuffle(srow.data_ptr(), full.data_ptr(), 4, [1] * 9, [1] * 9, [1] * 9)
    with pytest.raises(lib.B200Error, match="element size"):
        lib.dimshuffle(srow.data_ptr(), full.data_ptr(), 3, [2], [1], [1])


@pytest.mark.parametrize("flex", [False, True])
def test_reorders_through_the_transformer(flex):
    """axes_with_order results that have to be materialised, a reorder of a sliced view, a
    reordered operand of an elementwise op over five non-mergeable axes, and an assignment
    between differently laid-out tensors (the reference runs the last one as a dimshuffle too,
    ngraph/transformers/gputransform.py:393-395)."""
    import ngraph_python_b200 as ng
    ax = lambda n, nm: ng.make_axis(n, name=nm)   # noqa: E731
    A, B, C, D, E = ax(6, "A"), ax(5, "B"), ax(40, "C"), ax(3, "D"), ax(36, "E")
    rng = np.random.RandomState(0)
    # (a maximum just under a power of two would let the exponent manager try one more bit after
    # the first call and fall back two when that saturates: keep clear of the boundary)
    xv = rng.uniform(-0.8, 0.8, (6, 5, 40, 3, 36)).astype(np.float32)
    yv = rng.uniform(-0.8, 0.8, (36, 40, 6, 3, 5)).astype(np.float32)
    t = ng.transformers.allocate_transformer("b200", flex=flex)
    x = ng.placeholder([A, B, C, D, E])
    y = ng.placeholder([E, C, A, D, B])
    keep = ng.persistent_tensor([E, C, A, D, B], initial_value=0.)
    c1 = t.computation(ng.value_of(ng.axes_with_order(x, [E, D, C, B, A])), x)
    c2 = t.computation(ng.tanh(x) * ng.axes_with_order(y, [A, B, C, D, E]), x, y)
    sl = ng.tensor_slice(x, [slice(1, 5), slice(None), slice(0, 40, 2), slice(None), slice(None)])
    c3 = t.computation(ng.value_of(ng.axes_with_order(sl, list(reversed(list(sl.axes))))), x)
    c4 = t.computation(ng.sequential([ng.assign(keep, ng.axes_with_order(x, [E, C, A, D, B])),
                                      keep * 2.0]), x)
    t.initialize()
    assert [s.kind for s in c1.steps] == ["dimshuffle"]
    assert "dimshuffle" in [s.kind for s in c2.steps]
    assert [s.kind for s in c3.steps] == ["dimshuffle"]
    tol = dict(rtol=0, atol=2.0 ** -14) if flex else dict(rtol=0, atol=0)
    np.testing.assert_allclose(c1(xv), np.transpose(xv, (4, 3, 2, 1, 0)), **tol)
    want2 = np.tanh(xv) * np.transpose(yv, (2, 4, 1, 3, 0))
    np.testing.assert_allclose(c2(xv, yv), want2, rtol=1e-5, atol=2.0 ** -13 if flex else 1e-6)
    np.testing.assert_allclose(c3(xv), np.transpose(xv[1:5, :, 0:40:2], (4, 3, 2, 1, 0)), **tol)
    np.testing.assert_allclose(c4(xv), 2.0 * np.transpose(xv, (4, 2, 0, 3, 1)),
                               rtol=0, atol=2.0 ** -12 if flex else 0)
    t.close()


@pytest.mark.parametrize("perm", list(itertools.permutations(range(3))))
def test_every_3d_permutation_fp32(perm):
    import ngraph_python_b200 as ng
    axes = [ng.make_axis(n, name=nm) for n, nm in ((34, "A"), (65, "B"), (48, "C"))]
    x = ng.placeholder(axes)
    t = ng.transformers.allocate_transformer("b200")
    comp = t.computation(ng.value_of(ng.axes_with_order(x, [axes[i] for i in perm])), x)
    xv = np.random.RandomState(4).standard_normal((34, 65, 48)).astype(np.float32)
    assert np.array_equal(comp(xv), np.transpose(xv, perm))
    t.close()
