"""Graph cases shared by the fixture generator (run against the reference's CPU transformer) and
by the parity tests (run against the b200 transformer).  Every builder takes the `ng` namespace to
build with -- the reference's `ngraph` or `ngraph_python_b200` -- and returns
(outputs, parameters, input arrays); inputs are seeded so both sides see the same numbers.
"""
import numpy as np

from ngraph_python_b200.configs import (_conv_grad_ops, _conv_params, _rng, momentum_update,  # noqa: F401
                                         resnet20, resnet_train_step)


def c2_fused(ng, rows=24, cols=2048):
    """benchmark configuration 2: y = tanh(a*x+b)*sigmoid(c); sum and maxabs over axis 1."""
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


def conv_basic(ng, C=16, K=32, H=12, W=10, N=32, R=3, S=3, pad=1, stride=1):
    """One convolution forward, C,D,H,W,N * C,T,R,S,K -> K,M,P,Q,N
    (tests/transformer_dependent/test_conv.py:55-89)."""
    P = (H + 2 * pad - R) // stride + 1
    Q = (W + 2 * pad - S) // stride + 1
    ax = lambda n, nm: ng.make_axis(n, name=nm)   # noqa: E731
    ax_i = [ax(C, "C"), ax(1, "D"), ax(H, "H"), ax(W, "W"), ax(N, "N")]
    ax_f = [ax_i[0], ax(1, "T"), ax(R, "R"), ax(S, "S"), ax(K, "K")]
    ax_o = [ax_f[4], ax(1, "M"), ax(P, "P"), ax(Q, "Q"), ax_i[4]]
    inputs = ng.placeholder(ax_i)
    filters = ng.placeholder(ax_f)
    out = ng.convolution(_conv_params(pad, stride), inputs, filters, axes=ax_o)
    r = _rng(10)
    vals = [r.standard_normal((C, 1, H, W, N)).astype(np.float32),
            (r.standard_normal((C, 1, R, S, K)) * 0.2).astype(np.float32)]
    return [out], [inputs, filters], vals


def conv_stride2_1x1(ng):
    return conv_basic(ng, C=32, K=64, H=16, W=16, N=32, R=1, S=1, pad=0, stride=2)


def conv_stride2_3x3(ng):
    return conv_basic(ng, C=3, K=16, H=9, W=11, N=32, R=3, S=3, pad=1, stride=2)


def conv_grads(ng, C=16, K=32, H=12, W=10, N=32, R=3, S=3, pad=1, stride=1):
    """Forward convolution and its two gradients for a given error tensor
    (tests/transformer_dependent/test_conv.py:55-89 checks the same three results)."""
    P = (H + 2 * pad - R) // stride + 1
    Q = (W + 2 * pad - S) // stride + 1
    ax = lambda n, nm: ng.make_axis(n, name=nm)   # noqa: E731
    ax_i = [ax(C, "C"), ax(1, "D"), ax(H, "H"), ax(W, "W"), ax(N, "N")]
    ax_f = [ax_i[0], ax(1, "T"), ax(R, "R"), ax(S, "S"), ax(K, "K")]
    ax_o = [ax_f[4], ax(1, "M"), ax(P, "P"), ax(Q, "Q"), ax_i[4]]
    inputs = ng.placeholder(ax_i)
    filters = ng.placeholder(ax_f)
    delta = ng.placeholder(ax_o)
    bprop_conv, update_conv = _conv_grad_ops(ng)
    out = ng.convolution(_conv_params(pad, stride), inputs, filters, axes=ax_o)
    gi = bprop_conv(delta, inputs, filters, out)
    gf = update_conv(delta, inputs, filters, out)
    r = _rng(12)
    vals = [r.standard_normal((C, 1, H, W, N)).astype(np.float32),
            (r.standard_normal((C, 1, R, S, K)) * 0.2).astype(np.float32),
            (r.standard_normal((K, 1, P, Q, N)) * 0.5).astype(np.float32)]
    return [out, gi, gf], [inputs, filters, delta], vals


def conv_grads_stride2(ng):
    return conv_grads(ng, C=8, K=16, H=9, W=11, N=32, R=3, S=3, pad=1, stride=2)


def conv3d_grads(ng, C=6, K=10, D=4, H=7, W=8, N=32, T=2, R=3, S=2, pad=(1, 2, 0), stride=(1, 2, 1),
                 dil=(1, 1, 2)):
    """A convolution with real depth axes (D, T, M > 1), asymmetric padding / stride and a dilated
    width, forward and both gradients: the reference's kernels are C,D,H,W,N x C,T,R,S,K throughout
    (ngraph/transformers/gpu/flex_conv.py:49-200), and its flex convolution test runs a depth-2
    image (tests/flex_tests/test_flexconv.py:33).  pad / stride / dil are (depth, height, width)."""
    ext = lambda x, f, p_, s_, d_: (x + 2 * p_ - d_ * (f - 1) - 1) // s_ + 1   # noqa: E731
    M, P, Q = [ext(x, f, p_, s_, d_) for x, f, p_, s_, d_ in zip((D, H, W), (T, R, S), pad, stride, dil)]
    ax = lambda n, nm: ng.make_axis(n, name=nm)   # noqa: E731
    ax_i = [ax(C, "C"), ax(D, "D"), ax(H, "H"), ax(W, "W"), ax(N, "N")]
    ax_f = [ax_i[0], ax(T, "T"), ax(R, "R"), ax(S, "S"), ax(K, "K")]
    ax_o = [ax_f[4], ax(M, "M"), ax(P, "P"), ax(Q, "Q"), ax_i[4]]
    inputs, filters, delta = ng.placeholder(ax_i), ng.placeholder(ax_f), ng.placeholder(ax_o)
    params = dict(pad_d=pad[0], pad_h=pad[1], pad_w=pad[2], str_d=stride[0], str_h=stride[1],
                  str_w=stride[2], dil_d=dil[0], dil_h=dil[1], dil_w=dil[2])
    bprop_conv, update_conv = _conv_grad_ops(ng)
    out = ng.convolution(params, inputs, filters, axes=ax_o)
    gi = bprop_conv(delta, inputs, filters, out)
    gf = update_conv(delta, inputs, filters, out)
    r = _rng(71)
    vals = [r.standard_normal((C, D, H, W, N)).astype(np.float32),
            (r.standard_normal((C, T, R, S, K)) * 0.3).astype(np.float32),
            r.standard_normal((K, M, P, Q, N)).astype(np.float32)]
    return [out, gi, gf], [inputs, filters, delta], vals


def mlp_forward(ng):
    """Forward pass of benchmark configuration 1: 784 -> 512 ReLU -> 512 ReLU -> 10 softmax, batch 128."""
    r = _rng(0)
    N = ng.make_axis(128, name="N")
    F = ng.make_axis(784, name="F")
    H1 = ng.make_axis(512, name="H1")
    H2 = ng.make_axis(512, name="H2")
    Y = ng.make_axis(10, name="Y")
    x = ng.placeholder([F, N])

    def dense(inp, out_ax, in_ax):
        w = ng.variable([out_ax, in_ax], initial_value=(
            r.standard_normal((out_ax.length, in_ax.length)) *
            np.sqrt(2.0 / in_ax.length)).astype(np.float32))
        b = ng.variable([out_ax], initial_value=np.zeros(out_ax.length, np.float32))
        return ng.dot(w, inp) + b
    h1 = ng.maximum(dense(x, H1, F), 0.0)
    h2 = ng.maximum(dense(h1, H2, H1), 0.0)
    logits = dense(h2, Y, H2)
    e = ng.exp(logits - ng.max(logits, reduction_axes=[Y]))
    p = e / ng.sum(e, reduction_axes=[Y])
    vals = [_rng(1).uniform(0, 1, (784, 128)).astype(np.float32)]
    return [p, logits], [x], vals


def resnet8_small(ng):
    """A one-block-per-stage cut of the same network on 16x16 images (fast fixture)."""
    return resnet20(ng, n=32, hw=16, blocks=1)


def mlp_train_step(ng, global_n=128, shard=None, dims=(64, 48, 32, 10), lr=0.05, digest=False):
    """One data-parallel SGD step of a 3-layer MLP with softmax cross-entropy, gradients written
    out by hand (benchmark configurations 1 and 5 in miniature).  Every replica sees `shard = (rank,
    world)` of the global batch, scales its gradients by 1/global batch (the reference's optimizer
    divides by the global batch size, ngraph/frontends/neon/optimizer.py:177-198) and sum-allreduces
    them; with one replica the allreduce is the identity.  Returns the post-step weights and the
    pre-step mean loss."""
    allreduce = getattr(ng, "allreduce", None) or (lambda x, reduce_func="sum": x)
    rank, world = shard or (0, 1)
    local_n = global_n // world
    r = _rng(0)
    Fd, H1d, H2d, Yd = dims
    N = ng.make_axis(local_n, name="N")
    F, H1, H2, Y = [ng.make_axis(d, name=nm) for d, nm in zip(dims, ("F", "H1", "H2", "Y"))]
    x = ng.placeholder([F, N])
    t = ng.placeholder([Y, N])

    def weights(out_ax, in_ax):
        w = ng.variable([out_ax, in_ax], initial_value=(
            r.standard_normal((out_ax.length, in_ax.length)) *
            np.sqrt(2.0 / in_ax.length)).astype(np.float32))
        b = ng.variable([out_ax], initial_value=(r.standard_normal(out_ax.length) *
                                                 0.1).astype(np.float32))
        return w, b
    W1, b1 = weights(H1, F)
    W2, b2 = weights(H2, H1)
    W3, b3 = weights(Y, H2)
    z1 = ng.dot(W1, x) + b1
    a1 = ng.maximum(z1, 0.0)
    z2 = ng.dot(W2, a1) + b2
    a2 = ng.maximum(z2, 0.0)
    z3 = ng.dot(W3, a2) + b3
    e = ng.exp(z3 - ng.max(z3, reduction_axes=[Y]))
    p = e / ng.sum(e, reduction_axes=[Y])
    inv_n = 1.0 / global_n
    loss = allreduce(ng.sum(ng.negative(ng.sum(t * ng.log(p), reduction_axes=[Y])),
                            reduction_axes=[N]) * inv_n)
    dz3 = (p - t) * inv_n
    dW3 = ng.dot(dz3, a2)                      # [Y, H2], contracts N
    db3 = ng.sum(dz3, reduction_axes=[N])
    da2 = ng.dot(W3, dz3)                      # [H2, N], contracts Y
    dz2 = da2 * ng.greater(z2, 0.0)
    dW2 = ng.dot(dz2, a1)
    db2 = ng.sum(dz2, reduction_axes=[N])
    da1 = ng.dot(W2, dz2)
    dz1 = da1 * ng.greater(z1, 0.0)
    dW1 = ng.dot(dz1, x)
    db1 = ng.sum(dz1, reduction_axes=[N])
    updates = []
    for w, g in ((W3, dW3), (b3, db3), (W2, dW2), (b2, db2), (W1, dW1), (b1, db1)):
        updates.append(ng.assign(w, w - lr * allreduce(g)))
    step = ng.sequential(updates + [loss])
    outs = [step, W1, W2, W3, b3]
    if digest:
        # the biases of the first layers instead of their large weight matrices (their gradients
        # pass through the same back-propagation; keeps the fixture small)
        outs = [step, b1, b2, W3, b3]
    rng = _rng(3)
    xs = rng.uniform(0, 1, (Fd, global_n)).astype(np.float32)
    labels = np.eye(Yd, dtype=np.float32)[rng.randint(0, Yd, global_n)].T.copy()
    lo, hi = rank * local_n, (rank + 1) * local_n
    return outs, [x, t], [np.ascontiguousarray(xs[:, lo:hi]), np.ascontiguousarray(labels[:, lo:hi])]


def mlp_c1_train_step(ng, shard=None):
    """benchmark configuration 1 at full size: 784-512-512-10, batch 128, one SGD step (lr 0.01)."""
    return mlp_train_step(ng, global_n=128, shard=shard, dims=(784, 512, 512, 10), lr=0.01,
                          digest=True)


def batchnorm_train(ng, C=16, H=8, W=8, N=32, rho=0.9, eps=1e-3):
    """BatchNormalization in training mode as the reference's layer composes it
    (ngraph/frontends/neon/layer.py:1244-1256): batch mean and variance per channel, the running
    statistics updated in place, the batch normalised with gamma and beta.  The value returned
    also contains the inference formula evaluated on the running statistics AFTER their update,
    so the in-place assignments are part of what is compared."""
    r = _rng(21)
    ax = lambda n, nm: ng.make_axis(n, name=nm)   # noqa: E731
    Cx = ax(C, "C")
    x = ng.placeholder([Cx, ax(1, "D"), ax(H, "H"), ax(W, "W"), ax(N, "N")])
    gamma = ng.variable([Cx], initial_value=r.uniform(0.5, 1.5, C).astype(np.float32))
    beta = ng.variable([Cx], initial_value=r.uniform(-0.5, 0.5, C).astype(np.float32))
    gmean = ng.persistent_tensor(axes=[Cx], initial_value=0.)
    gvar = ng.persistent_tensor(axes=[Cx], initial_value=1.)
    xmean = ng.mean(x, out_axes=[Cx])
    xvar = ng.variance(x, out_axes=[Cx])
    y_train = gamma * ((x - xmean) * ng.reciprocal(ng.sqrt(xvar + eps))) + beta
    y_infer = gamma * ((x - gmean) * ng.reciprocal(ng.sqrt(gvar + eps))) + beta
    out = ng.sequential([
        ng.assign(gmean, gmean * rho + xmean * (1.0 - rho)),
        ng.assign(gvar, gvar * rho + xvar * (1.0 - rho)),
        y_train + 0.5 * y_infer,
    ])
    vals = [(_rng(22).standard_normal((C, 1, H, W, N)) * 1.7 + 0.4).astype(np.float32)]
    return [out], [x], vals


def pool_max(ng, C=12, H=9, W=11, N=32, R=3, S=3, pad=1, stride=2):
    """Max pooling forward with padding and stride (the reference's PoolingOp, np.max over the
    in-image part of each window, ngraph/transformers/cpu/cpuengine.py:286-300)."""
    ax = lambda n, nm: ng.make_axis(n, name=nm)   # noqa: E731
    P = (H + 2 * pad - R) // stride + 1
    Q = (W + 2 * pad - S) // stride + 1
    Cx, D, Nx = ax(C, "C"), ax(1, "D"), ax(N, "N")
    x = ng.placeholder([Cx, D, ax(H, "H"), ax(W, "W"), Nx])
    pool = dict(op="max", J=1, T=1, R=R, S=S, pad_c=0, pad_d=0, pad_h=pad, pad_w=pad,
                str_c=1, str_d=1, str_h=stride, str_w=stride)
    out = ng.pooling(pool, x, axes=[Cx, D, ax(P, "P"), ax(Q, "Q"), Nx])
    vals = [_rng(31).standard_normal((C, 1, H, W, N)).astype(np.float32)]
    return [ng.tanh(out) + out], [x], vals


def _pool_grad_op(ng):
    """bprop_pool: the reference keeps BpropPoolOp in ngraph.op_graph.pooling."""
    if hasattr(ng, "bprop_pool"):
        return ng.bprop_pool
    from ngraph.op_graph.pooling import BpropPoolOp
    return lambda delta, inputs, fprop: BpropPoolOp(delta, inputs, fprop)


def pool_grads(ng, op="max", C=6, H=9, W=11, N=32, R=3, S=3, pad=1, stride=2):
    """Pooling forward and its input gradient for a given error tensor, overlapping windows
    (3x3, stride 2, padding 1): what the reference's autodiff emits for a pooling layer."""
    ax = lambda n, nm: ng.make_axis(n, name=nm)   # noqa: E731
    P = (H + 2 * pad - R) // stride + 1
    Q = (W + 2 * pad - S) // stride + 1
    Cx, D, Nx = ax(C, "C"), ax(1, "D"), ax(N, "N")
    x = ng.placeholder([Cx, D, ax(H, "H"), ax(W, "W"), Nx])
    delta = ng.placeholder([Cx, D, ax(P, "P"), ax(Q, "Q"), Nx])
    pool = dict(op=op, J=1, T=1, R=R, S=S, pad_c=0, pad_d=0, pad_h=pad, pad_w=pad,
                str_c=1, str_d=1, str_h=stride, str_w=stride)
    out = ng.pooling(pool, x, axes=delta.axes)
    gi = _pool_grad_op(ng)(delta, x, out)
    r = _rng(41)
    vals = [r.standard_normal((C, 1, H, W, N)).astype(np.float32),
            r.standard_normal((C, 1, P, Q, N)).astype(np.float32)]
    return [out, gi], [x, delta], vals


def pool_grads_avg(ng):
    return pool_grads(ng, op="avg")


def lut_embedding(ng, V=50, F=24, n=40, pad_idx=0, lut_axis=0):
    """Embedding lookup and the gradient of the table for a given error tensor, with repeated
    indices and a padding index (the reference's LookupTableOp / update_lut,
    ngraph/op_graph/lookuptable.py; tests/transformer_dependent/test_lookuptable.py builds the
    same pair)."""
    ax = lambda k, nm: ng.make_axis(k, name=nm)   # noqa: E731
    Vx, Fx, Nx = ax(V, "V"), ax(F, "F"), ax(n, "NI")
    r = _rng(51)
    lut_axes = [Vx, Fx] if lut_axis == 0 else [Fx, Vx]
    out_axes = [Nx, Fx] if lut_axis == 0 else [Fx, Nx]
    lut = ng.placeholder(lut_axes)
    idx = ng.placeholder([Nx])
    delta = ng.placeholder(out_axes)
    out = ng.lookuptable(lut, idx, out_axes, pad_idx=pad_idx)
    if hasattr(ng, "lookuptable_update"):
        grad = ng.lookuptable_update(delta, lut, idx, out)
    else:
        from ngraph.op_graph.lookuptable import lookuptable_update
        grad = lookuptable_update(delta, lut, idx, out)
    idx_val = r.randint(0, V, n).astype(np.float32)
    if pad_idx is not None:
        idx_val[::7] = pad_idx
    idx_val[3::5] = idx_val[3]                       # repeats
    vals = [r.standard_normal([a.length for a in lut_axes]).astype(np.float32), idx_val,
            r.standard_normal([a.length for a in out_axes]).astype(np.float32)]
    return [out * 2.0, grad], [lut, idx, delta], vals


def lut_embedding_axis1(ng):
    return lut_embedding(ng, V=33, F=20, n=48, pad_idx=None, lut_axis=1)


def slice_views(ng):
    """Sliced views read and written: a strided window of the input, an integer index that drops
    an axis, and an assignment into a slice of a persistent tensor that is read back afterwards
    (what the reference's adjoint of a slice does, ngraph/op_graph/op_graph.py: UnsliceOp)."""
    ax = lambda n, nm: ng.make_axis(n, name=nm)   # noqa: E731
    A, B, Cx = ax(6, "A"), ax(10, "B"), ax(3, "C")
    x = ng.placeholder([A, B, Cx])
    temp = ng.persistent_tensor(axes=[A, B], initial_value=0.)
    window = [slice(1, 5), slice(2, 7)]
    plane = ng.tensor_slice(x, [slice(None), slice(None), 1])            # (A, B): axis C dropped
    part = ng.tensor_slice(plane, window)                                # (4, 5) window
    out = ng.sequential([
        ng.assign(temp, plane * 0.25),
        ng.assign(ng.tensor_slice(temp, window), ng.tanh(part) + 3.0),
        temp * 2.0,
    ])
    vals = [_rng(61).standard_normal((6, 10, 3)).astype(np.float32)]
    return [out, ng.sum(part, reduction_axes=[part.axes[1]])], [x], vals


CASES = {
    "slice_views": slice_views,
    "lut_embedding": lut_embedding,
    "lut_embedding_axis1": lut_embedding_axis1,
    "pool_grads": pool_grads,
    "pool_grads_avg": pool_grads_avg,
    "pool_max": pool_max,
    "batchnorm_train": batchnorm_train,
    "mlp_train_step": mlp_train_step,
    "mlp_c1_train_step": mlp_c1_train_step,
    "resnet_train_step": resnet_train_step,
    "conv_basic": conv_basic,
    "conv_stride2_1x1": conv_stride2_1x1,
    "conv_stride2_3x3": conv_stride2_3x3,
    "conv_grads": conv_grads,
    "conv_grads_stride2": conv_grads_stride2,
    "conv3d_grads": conv3d_grads,
    "mlp_forward": mlp_forward,
    "resnet20": resnet20,
    "resnet8_small": resnet8_small,
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
REPEAT = {"slice_views": 2, "batchnorm_train": 2, "assign_sequence": 2, "mlp_train_step": 2, "mlp_c1_train_step": 2,
          "resnet_train_step": 2}
