"""The benchmark configurations as graphs: ResNet-20 inference (configuration 4) and one
data-parallel training step of the same network (configuration 5).

Every builder takes the namespace to build with -- the reference's `ngraph` or this package --
and returns (outputs, parameters, input arrays), so the same function gives the graph the
reference's CPU transformer evaluates and the graph the b200 transformer runs.  The parity
fixtures (tests/golden/) and bench.py both build from here.
"""
import numpy as np


def _rng(seed):
    return np.random.RandomState(seed)


def _conv_params(pad, stride):
    return dict(pad_d=0, pad_h=pad, pad_w=pad, str_d=1, str_h=stride, str_w=stride,
                dil_d=1, dil_h=1, dil_w=1)


def _conv_grad_ops(ng):
    """bprop_conv / update_conv: the reference keeps them in ngraph.op_graph.convolution, outside
    its ng namespace."""
    if hasattr(ng, "bprop_conv"):
        return ng.bprop_conv, ng.update_conv
    from ngraph.op_graph.convolution import bprop_conv, update_conv
    return bprop_conv, update_conv


def resnet20(ng, n=32, hw=32, widths=(16, 32, 64), blocks=3):
    """ResNet-20 inference (benchmark configuration 4): 3 stages of 3 basic blocks, 3x3 convolutions,
    batch norm folded into per-channel biases, a 1x1 projection on the first block of every stage,
    8x8 average pool, 10-way linear, softmax.  22 convolutions, He-initialised from seed 0."""
    r = _rng(0)
    ax = lambda nlen, nm: ng.make_axis(nlen, name=nm)   # noqa: E731
    N = ax(n, "N")
    D = ax(1, "D")
    T = ax(1, "T")
    C3 = ax(3, "C3")
    x = ng.placeholder([C3, D, ax(hw, "H0"), ax(hw, "W0"), N])
    counter = [0]

    def conv(inp, cout_axis, k, stride, out_sp):
        """inp axes (Cin, D, H, W, N) -> (cout_axis, D, H', W', N) with bias."""
        i = counter[0]
        counter[0] += 1
        cin = inp.axes[0]
        Kt = ax(cout_axis.length, "K%d" % i)
        fan_in = cin.length * k * k
        f = ng.variable([cin, T, ax(k, "R%d" % i), ax(k, "S%d" % i), Kt],
                        initial_value=(r.standard_normal((cin.length, 1, k, k, Kt.length)) *
                                       np.sqrt(2.0 / fan_in)).astype(np.float32))
        b = ng.variable([cout_axis], initial_value=(r.standard_normal(cout_axis.length) *
                                                    0.05).astype(np.float32))
        o = ng.convolution(_conv_params(k // 2, stride), inp, f,
                           axes=[Kt, ax(1, "M%d" % i), out_sp[0], out_sp[1], N])
        o = ng.cast_axes(o, [cout_axis, D, out_sp[0], out_sp[1], N])
        return o + b

    size = hw
    sp = (ax(size, "H%d" % size), ax(size, "W%d" % size))
    cur = ng.maximum(conv(x, ax(widths[0], "C%d" % widths[0]), 3, 1, sp), 0.0)
    for s, width in enumerate(widths):
        c_axis = ax(width, "C%d" % width)
        for b in range(blocks):
            stride = 2 if (b == 0 and s > 0) else 1
            if stride == 2:
                size //= 2
                sp = (ax(size, "H%d" % size), ax(size, "W%d" % size))
            y = ng.maximum(conv(cur, c_axis, 3, stride, sp), 0.0)
            y = conv(y, c_axis, 3, 1, sp)
            shortcut = conv(cur, c_axis, 1, stride, sp) if b == 0 else cur
            cur = ng.maximum(y + shortcut, 0.0)
    pool = dict(op="avg", J=1, T=1, R=size, S=size, pad_c=0, pad_d=0, pad_h=0, pad_w=0,
                str_c=1, str_d=1, str_h=1, str_w=1)
    pooled = ng.pooling(pool, cur, axes=[cur.axes[0], D, ax(1, "PP"), ax(1, "QQ"), N])
    Y = ax(10, "Y")
    w = ng.variable([Y, cur.axes[0]], initial_value=(
        r.standard_normal((10, widths[-1])) * np.sqrt(2.0 / widths[-1])).astype(np.float32))
    by = ng.variable([Y], initial_value=np.zeros(10, np.float32))
    logits = ng.dot(w, pooled) + by
    e = ng.exp(logits - ng.max(logits, reduction_axes=[Y]))
    p = e / ng.sum(e, reduction_axes=[Y])
    vals = [_rng(1).standard_normal((3, 1, hw, hw, n)).astype(np.float32)]
    return [p, logits], [x], vals


class _Tape(object):
    """Reverse-mode bookkeeping for the hand-written gradients of resnet_train_step: forward helpers
    record (output, backward function); backward() walks them in reverse and sums what arrives at
    each tensor."""

    def __init__(self):
        self.entries = []
        self.grads = {}
        self.param_grads = []          # (variable, gradient) in the order they are produced

    def record(self, out, fn):
        self.entries.append((out, fn))

    def add(self, t, g):
        k = id(t)
        self.grads[k] = g if k not in self.grads else self.grads[k] + g

    def backward(self, out, dout):
        self.grads[id(out)] = dout
        for o, fn in reversed(self.entries):
            g = self.grads.get(id(o))
            if g is not None:
                fn(g)


def momentum_update(ng, variable, grad, lr, momentum, wdecay=0.0):
    """GradientDescentMomentum.variable_update with its Kahan-compensated weight update
    (ngraph/frontends/neon/optimizer.py:285-310): four persistent tensors per variable."""
    zeros = lambda: ng.persistent_tensor(axes=variable.axes, initial_value=0.)   # noqa: E731
    velocity, kahan_c, kahan_y, kahan_t = zeros(), zeros(), zeros(), zeros()
    step = -lr * (grad + wdecay * variable) if wdecay else -lr * grad
    return ng.sequential([
        ng.assign(velocity, velocity * momentum + step),
        ng.assign(kahan_y, velocity - kahan_c),
        ng.assign(kahan_t, variable + kahan_y),
        ng.assign(kahan_c, (kahan_t - variable) - kahan_y),
        ng.assign(variable, kahan_t),
    ])


def resnet_train_step(ng, global_n=32, shard=None, hw=16, widths=(16, 32, 64), blocks=1, lr=0.1,
                      momentum=0.9):
    """One data-parallel training step of the ResNet of resnet20() (benchmark configuration 5): softmax
    cross-entropy, gradients written out with bprop_conv / update_conv, sum-allreduce of every
    gradient (already divided by the GLOBAL batch, as the reference's optimizer divides,
    ngraph/frontends/neon/optimizer.py:177-198), momentum SGD with Kahan summation.
    Returns [step (-> mean loss before the update), first filters, last filters, linear weights]."""
    allreduce = getattr(ng, "allreduce", None) or (lambda x, reduce_func="sum": x)
    bprop_conv, update_conv = _conv_grad_ops(ng)
    rank, world = shard or (0, 1)
    n = global_n // world
    r = _rng(0)
    ax = lambda nlen, nm: ng.make_axis(nlen, name=nm)   # noqa: E731
    N, D, T = ax(n, "N"), ax(1, "D"), ax(1, "T")
    x = ng.placeholder([ax(3, "C3"), D, ax(hw, "H0"), ax(hw, "W0"), N])
    tape = _Tape()
    counter = [0]
    params = []

    def conv(inp, cout_axis, k, stride, out_sp, need_dinp=True):
        i = counter[0]
        counter[0] += 1
        cin = inp.axes[0]
        Kt = ax(cout_axis.length, "K%d" % i)
        fan_in = cin.length * k * k
        f = ng.variable([cin, T, ax(k, "R%d" % i), ax(k, "S%d" % i), Kt],
                        initial_value=(r.standard_normal((cin.length, 1, k, k, Kt.length)) *
                                       np.sqrt(2.0 / fan_in)).astype(np.float32))
        b = ng.variable([cout_axis], initial_value=(r.standard_normal(cout_axis.length) *
                                                    0.05).astype(np.float32))
        params.extend([f, b])
        conv_axes = [Kt, ax(1, "M%d" % i), out_sp[0], out_sp[1], N]
        o = ng.convolution(_conv_params(k // 2, stride), inp, f, axes=conv_axes)
        out = ng.cast_axes(o, [cout_axis, D, out_sp[0], out_sp[1], N]) + b

        def back(d):
            tape.param_grads.append((b, ng.sum(d, reduction_axes=[D, out_sp[0], out_sp[1], N])))
            dk = ng.cast_axes(d, conv_axes)
            tape.param_grads.append((f, update_conv(dk, inp, f, o)))
            if need_dinp:
                tape.add(inp, bprop_conv(dk, inp, f, o))
        tape.record(out, back)
        return out

    def relu(pre):
        out = ng.maximum(pre, 0.0)
        tape.record(out, lambda d: tape.add(pre, d * ng.greater(pre, 0.0)))
        return out

    def add(a, b_):
        out = a + b_

        def back(d):
            tape.add(a, d)
            tape.add(b_, d)
        tape.record(out, back)
        return out

    size = hw
    sp = (ax(size, "H%d" % size), ax(size, "W%d" % size))
    cur = relu(conv(x, ax(widths[0], "C%d" % widths[0]), 3, 1, sp, need_dinp=False))
    for s_, width in enumerate(widths):
        c_axis = ax(width, "C%d" % width)
        for b_ in range(blocks):
            stride = 2 if (b_ == 0 and s_ > 0) else 1
            if stride == 2:
                size //= 2
                sp = (ax(size, "H%d" % size), ax(size, "W%d" % size))
            y = relu(conv(cur, c_axis, 3, stride, sp))
            y = conv(y, c_axis, 3, 1, sp)
            shortcut = conv(cur, c_axis, 1, stride, sp) if b_ == 0 else cur
            cur = relu(add(y, shortcut))
    pool = dict(op="avg", J=1, T=1, R=size, S=size, pad_c=0, pad_d=0, pad_h=0, pad_w=0,
                str_c=1, str_d=1, str_h=1, str_w=1)
    PP, QQ = ax(1, "PP"), ax(1, "QQ")
    feat = cur
    pooled = ng.pooling(pool, feat, axes=[feat.axes[0], D, PP, QQ, N])

    def pool_back(d):
        flat = ng.sum(d, reduction_axes=[PP, QQ]) * (1.0 / (size * size))
        tape.add(feat, ng.broadcast(flat, feat.axes))
    tape.record(pooled, pool_back)
    Y = ax(10, "Y")
    w = ng.variable([Y, feat.axes[0]], initial_value=(
        r.standard_normal((10, widths[-1])) * np.sqrt(2.0 / widths[-1])).astype(np.float32))
    by = ng.variable([Y], initial_value=np.zeros(10, np.float32))
    params.extend([w, by])
    logits = ng.dot(w, pooled) + by

    def dense_back(d):
        tape.param_grads.append((by, ng.sum(d, reduction_axes=[D, PP, QQ, N])))
        tape.param_grads.append((w, ng.dot(d, pooled)))
        tape.add(pooled, ng.dot(w, d))
    tape.record(logits, dense_back)
    t = ng.placeholder([Y, N])
    e = ng.exp(logits - ng.max(logits, reduction_axes=[Y]))
    p = e / ng.sum(e, reduction_axes=[Y])
    inv_n = 1.0 / global_n
    loss = allreduce(ng.sum(ng.negative(t * ng.log(p)), reduction_axes=[Y, D, PP, QQ, N]) * inv_n)
    tape.backward(logits, (p - t) * inv_n)
    # every gradient is evaluated before the first weight changes, as the reference's optimizer
    # orders them (ng.sequential([grads, updates, ...]), ngraph/frontends/neon/optimizer.py:203-211)
    grads = [allreduce(g) for _, g in tape.param_grads]
    updates = [momentum_update(ng, v, g, lr, momentum)
               for (v, _), g in zip(tape.param_grads, grads)]
    step = ng.sequential(grads + updates + [loss])
    outs = [step, params[0], params[-4], w]
    rng = _rng(3)
    xs = rng.standard_normal((3, 1, hw, hw, global_n)).astype(np.float32)
    labels = np.eye(10, dtype=np.float32)[rng.randint(0, 10, global_n)].T.copy()
    lo, hi = rank * n, (rank + 1) * n
    return outs, [x, t], [np.ascontiguousarray(xs[..., lo:hi]), np.ascontiguousarray(labels[:, lo:hi])]
