"""Graph cases shared by the fixture generator (run against the reference's CPU transformer) and
by the parity tests (run against the b200 transformer).  Every builder takes the `ng` namespace to
build with -- the reference's `ngraph` or `ngraph_python_b200` -- and returns
(outputs, parameters, input arrays); inputs are seeded so both sides see the same numbers.
"""
import numpy as np


def _rng(seed):
    return np.random.RandomState(seed)


def c2_fused(ng, rows=24, cols=2048):
    """BASELINE config 2: y = tanh(a*x+b)*sigmoid(c); sum and maxabs over axis 1."""
    R = ng.make_axis(rows, name="R")
    C = ng.make_axis(cols, name="C")
    ph = [ng.placeholder([R, C]) for _ in range(4)]
    x, a, b, c = ph
    y = ng.tanh(a * x + b) * ng.sigmoid(c)
    s = ng.sum(y, reduction_axes=[C])
    m = ng.max(ng.absolute(y), reduction_axes=[C])
    r = _rng(0)
    vals = [r.standard_normal((rows, cols)).astype(np.float32) for _ in range(4)]
    return [y, s, m], ph, vals


def ew_4d(ng):
    """4-d elementwise chain (tests/transformer_dependent/test_kernel_generator.py:43-76)."""
    axes = [ng.make_axis(n, name=nm) for n, nm in ((16, "A"), (16, "B"), (8, "C"), (8, "D"))]
    x = ng.placeholder(axes)
    y = ng.placeholder(axes)
    out = ng.exp(ng.negative(ng.absolute(x))) + ng.sqrt(ng.absolute(y)) * 0.5 - x / (y * y + 1.0)
    r = _rng(1)
    vals = [r.uniform(-1, 1, (16, 16, 8, 8)).astype(np.float32) for _ in range(2)]
    return [out], [x, y], vals


def reduce_4d_axis1(ng):
    """Reduction over a middle axis of a 4-d tensor (test_kernel_generator.py:79-113)."""
    axes = [ng.make_axis(n, name=nm) for n, nm in ((16, "A"), (24, "B"), (8, "C"), (8, "D"))]
    x = ng.placeholder(axes)
    out = [ng.sum(x, reduction_axes=[axes[1]]), ng.max(x, reduction_axes=[axes[1]]),
           ng.min(x, reduction_axes=[axes[1]])]
    vals = [_rng(2).uniform(-1, 1, (16, 24, 8, 8)).astype(np.float32)]
    return out, [x], vals


def reduce_4d_axis3(ng):
    """Reduction over the innermost axis (test_kernel_generator.py:116-150)."""
    axes = [ng.make_axis(n, name=nm) for n, nm in ((16, "A"), (16, "B"), (8, "C"), (40, "D"))]
    x = ng.placeholder(axes)
    out = [ng.sum(x, reduction_axes=[axes[3]]), ng.prod(x * 0.5 + 1.0, reduction_axes=[axes[3]]),
           ng.argmax(x, reduction_axes=[axes[3]]), ng.argmin(x, reduction_axes=[axes[3]])]
    vals = [_rng(3).uniform(-1, 1, (16, 16, 8, 40)).astype(np.float32)]
    return out, [x], vals


def recip_add_sum(ng):
    """Chained reciprocal + add + sum (test_kernel_generator.py:153-176)."""
    M = ng.make_axis(32, name="M")
    N = ng.make_axis(96, name="N")
    x = ng.placeholder([M, N])
    y = ng.placeholder([M, N])
    out = ng.sum(ng.reciprocal(x) + y, reduction_axes=[N])
    r = _rng(4)
    vals = [r.uniform(0.5, 2, (32, 96)).astype(np.float32),
            r.uniform(-1, 1, (32, 96)).astype(np.float32)]
    return [out], [x, y], vals


def broadcast_bias(ng):
    """Row- and column-broadcast operands, scalar constants, full reduction."""
    K = ng.make_axis(48, name="K")
    N = ng.make_axis(128, name="N")
    x = ng.placeholder([K, N])
    bias = ng.placeholder([K])
    gain = ng.placeholder([N])
    y = ng.maximum(x + bias, 0.0) * gain
    total = ng.sum(y, reduction_axes=[K, N])
    colsum = ng.sum(y, reduction_axes=[K])
    r = _rng(5)
    vals = [r.standard_normal((48, 128)).astype(np.float32),
            r.standard_normal((48,)).astype(np.float32),
            r.uniform(0.5, 1.5, (128,)).astype(np.float32)]
    return [y, total, colsum], [x, bias, gain], vals


def softmax_xent(ng):
    """Softmax + cross-entropy tail of the MLP / ResNet graphs."""
    Y = ng.make_axis(10, name="Y")
    N = ng.make_axis(128, name="N")
    x = ng.placeholder([Y, N])
    t = ng.placeholder([Y, N])
    xs = x - ng.max(x, reduction_axes=[Y])
    e = ng.exp(xs)
    p = e / ng.sum(e, reduction_axes=[Y])
    loss = ng.negative(ng.sum(t * ng.safelog(p), reduction_axes=[Y]))
    mean_loss = ng.sum(loss, reduction_axes=[N]) / 128.0
    r = _rng(6)
    logits = (r.standard_normal((10, 128)) * 3).astype(np.float32)
    labels = np.eye(10, dtype=np.float32)[r.randint(0, 10, 128)].T.copy()
    return [p, loss, mean_loss], [x, t], [logits, labels]


def unary_binary_sweep(ng):
    """Every elementwise op of the table (ngraph/transformers/gputransform.py:124-275)."""
    A = ng.make_axis(37, name="A")
    B = ng.make_axis(53, name="B")
    x = ng.placeholder([A, B])
    y = ng.placeholder([A, B])
    pos = ng.absolute(x) + 0.5
    outs = [ng.negative(x), ng.absolute(x), ng.sqrt(pos), ng.square(x), ng.exp(x), ng.log(pos),
            ng.reciprocal(pos), ng.tanh(x), ng.sign(x), ng.sin(x), ng.cos(x), ng.safelog(pos - 0.5),
            x + y, x - y, x * y, x / (ng.absolute(y) + 0.5), ng.maximum(x, y), ng.minimum(x, y),
            ng.power(pos, y), ng.equal(x, y), ng.not_equal(x, y), ng.less(x, y),
            ng.less_equal(x, y), ng.greater(x, y), ng.greater_equal(x, y)]
    r = _rng(7)
    vals = [r.standard_normal((37, 53)).astype(np.float32) * 2,
            r.standard_normal((37, 53)).astype(np.float32)]
    vals[1][3, :10] = vals[0][3, :10]     # some equal pairs
    return outs, [x, y], vals


def assign_sequence(ng):
    """In-place update of a variable inside a sequential, value read back afterwards."""
    A = ng.make_axis(33, name="A")
    B = ng.make_axis(65, name="B")
    g = ng.placeholder([A, B])
    w = ng.variable([A, B], initial_value=_rng(8).standard_normal((33, 65)).astype(np.float32))
    upd = ng.sequential([ng.assign(w, w - 0.1 * g), ng.sum(w * w, reduction_axes=[A, B])])
    vals = [_rng(9).standard_normal((33, 65)).astype(np.float32)]
    return [upd], [g], vals


CASES = {
    "c2_fused": c2_fused,
    "ew_4d": ew_4d,
    "reduce_4d_axis1": reduce_4d_axis1,
    "reduce_4d_axis3": reduce_4d_axis3,
    "recip_add_sum": recip_add_sum,
    "broadcast_bias": broadcast_bias,
    "softmax_xent": softmax_xent,
    "unary_binary_sweep": unary_binary_sweep,
    "assign_sequence": assign_sequence,
}
# cases evaluated twice in a row (state carried by variables)
REPEAT = {"assign_sequence": 2}
