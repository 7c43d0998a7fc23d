"""Graph-building surface for the B200 transformer.

Mirrors the part of the reference's `ng.*` op surface that the hot path uses
(ngraph/__init__.py:23-89, ngraph/op_graph/op_graph.py, ngraph/op_graph/axes.py): named axes,
placeholders / variables / constants, elementwise ops with broadcasting by axis name,
reductions, dot, convolution, pooling, assign and sequential.  Names, argument meaning and error
behaviour follow the reference so that tests read like the reference's own; autodiff, serde and
the frontends are not part of this package.
"""
import itertools
import numbers

import numpy as np

_axis_counter = itertools.count()


class Axis(object):
    """A named dimension (ngraph/op_graph/axes.py: make_axis).  Two axes match when name and
    length are equal."""

    def __init__(self, length, name=None):
        if name is None:
            name = "Axis_%d" % next(_axis_counter)
        self.name = name
        self._length = None if length is None else int(length)

    @property
    def length(self):
        return self._length

    @length.setter
    def length(self, value):
        self._length = int(value)

    @property
    def is_batch(self):
        return self.name == "N"

    def named(self, name):
        return Axis(self.length, name)

    def __eq__(self, other):
        return isinstance(other, Axis) and self.name == other.name and self.length == other.length

    def __ne__(self, other):
        return not self == other

    def __hash__(self):
        return hash((self.name, self._length))

    def __repr__(self):
        return "Axis(%s: %s)" % (self.name, self._length)


def make_axis(length=None, name=None, **kw):
    return Axis(length, name)


class Axes(object):
    """An ordered collection of axes (ngraph/op_graph/axes.py: Axes)."""

    def __init__(self, axes=None):
        if axes is None:
            axes = ()
        elif isinstance(axes, Axis):
            axes = (axes,)
        elif isinstance(axes, Axes):
            axes = axes._axes
        axes = tuple(axes)
        for a in axes:
            if not isinstance(a, Axis):
                raise ValueError("Axes must contain Axis objects, got %r" % (a,))
        names = [a.name for a in axes]
        if len(set(names)) != len(names):
            raise ValueError("The axes labels of a tensor cannot contain duplicates: %s" % names)
        self._axes = axes

    def __iter__(self):
        return iter(self._axes)

    def __len__(self):
        return len(self._axes)

    def __getitem__(self, i):
        if isinstance(i, slice):
            return Axes(self._axes[i])
        return self._axes[i]

    def __add__(self, other):
        other = make_axes(other)
        return Axes(self._axes + tuple(a for a in other if a not in self._axes))

    def __sub__(self, other):
        other = make_axes(other)
        return Axes(a for a in self._axes if a not in other._axes)

    def __and__(self, other):
        other = make_axes(other)
        return Axes(a for a in self._axes if a in other._axes)

    def __eq__(self, other):
        return isinstance(other, Axes) and self._axes == other._axes

    def __ne__(self, other):
        return not self == other

    def __hash__(self):
        return hash(self._axes)

    def __contains__(self, a):
        return a in self._axes

    def __repr__(self):
        return "Axes(%s)" % ", ".join("%s: %s" % (a.name, a.length) for a in self._axes)

    def index(self, a):
        return self._axes.index(a)

    def find_by_name(self, name):
        return Axes(a for a in self._axes if a.name == name)

    def is_equal_set(self, other):
        return set(self._axes) == set(make_axes(other)._axes)

    def is_sub_set(self, other):
        return set(self._axes) <= set(make_axes(other)._axes)

    @property
    def lengths(self):
        return tuple(a.length for a in self._axes)

    @property
    def size(self):
        return int(np.prod(self.lengths, dtype=np.int64)) if self._axes else 1

    def batch_axis(self):
        for a in self._axes:
            if a.is_batch:
                return a
        return None


def make_axes(axes=()):
    if isinstance(axes, Axes):
        return axes
    return Axes(axes)


# ---------------------------------------------------------------------------------------------
class Op(object):
    """Base of all graph nodes."""
    _counter = itertools.count()

    def __init__(self, args=(), axes=(), name=None, metadata=None):
        self.args = tuple(as_op(a) for a in args)
        self.axes = make_axes(axes)
        self.uid = next(Op._counter)
        self.name = name or "%s_%d" % (type(self).__name__, self.uid)
        self.metadata = dict(metadata or {})
        self.control_deps = []

    is_tensor_op = True
    is_device_op = True

    @property
    def shape(self):
        return self.axes.lengths

    def add_control_dep(self, op):
        if op is not self and op not in self.control_deps:
            self.control_deps.append(op)

    @property
    def all_deps(self):
        return list(self.args) + list(self.control_deps)

    # arithmetic sugar, as on the reference's TensorOp
    def __neg__(self):
        return negative(self)

    def __pos__(self):
        return self

    def __abs__(self):
        return absolute(self)

    def __add__(self, o):
        return add(self, o)

    def __radd__(self, o):
        return add(o, self)

    def __sub__(self, o):
        return subtract(self, o)

    def __rsub__(self, o):
        return subtract(o, self)

    def __mul__(self, o):
        return multiply(self, o)

    def __rmul__(self, o):
        return multiply(o, self)

    def __truediv__(self, o):
        return divide(self, o)

    def __rtruediv__(self, o):
        return divide(o, self)

    __div__ = __truediv__
    __rdiv__ = __rtruediv__

    def __pow__(self, o):
        return power(self, o)

    def __rpow__(self, o):
        return power(o, self)

    __hash__ = object.__hash__

    def __repr__(self):
        return "<%s %s %s>" % (type(self).__name__, self.name, self.axes)


class AssignableTensorOp(Op):
    """placeholder / variable / persistent tensor / constant
    (ngraph/op_graph/op_graph.py: AssignableTensorOp)."""
    is_device_op = False

    def __init__(self, axes, initial_value=None, is_input=False, is_persistent=False,
                 is_constant=False, is_trainable=False, is_placeholder=False, **kw):
        super(AssignableTensorOp, self).__init__((), axes, **kw)
        self.is_input = is_input
        self.is_persistent = is_persistent
        self.is_constant = is_constant
        self.is_trainable = is_trainable
        self.is_placeholder = is_placeholder
        if initial_value is not None and not callable(initial_value):
            initial_value = np.asarray(initial_value, dtype=np.float32)
            lengths = tuple(self.axes.lengths)
            if initial_value.shape not in ((), lengths):
                # the same elements up to axes of length 1, or a value that numpy broadcasts to
                # the axes (the reference hands initial values to numpy the same way)
                if tuple(n for n in initial_value.shape if n != 1) == \
                        tuple(n for n in lengths if n != 1):
                    initial_value = initial_value.reshape(lengths)
                else:
                    try:
                        initial_value = np.ascontiguousarray(np.broadcast_to(initial_value, lengths))
                    except ValueError:
                        raise ValueError("initial value shape %s does not match axes %s" %
                                         (initial_value.shape, self.axes))
        self.initial_value = initial_value

    @property
    def is_scalar_constant(self):
        return self.is_constant and len(self.axes) == 0

    def initial_array(self):
        v = self.initial_value
        if v is None:
            return None
        if callable(v):
            v = np.asarray(v(self.axes), dtype=np.float32)
        return np.ascontiguousarray(np.broadcast_to(v, self.axes.lengths), dtype=np.float32)


def placeholder(axes, dtype=None, initial_value=None, **kw):
    return AssignableTensorOp(make_axes(axes), initial_value, is_input=True, is_persistent=True,
                              is_placeholder=True, **kw)


def variable(axes, dtype=None, initial_value=None, **kw):
    return AssignableTensorOp(make_axes(axes), initial_value, is_input=True, is_persistent=True,
                              is_trainable=True, **kw)


def persistent_tensor(axes, dtype=None, initial_value=None, **kw):
    return AssignableTensorOp(make_axes(axes), initial_value, is_persistent=True, **kw)


def temporary(axes, dtype=None, initial_value=None, **kw):
    return AssignableTensorOp(make_axes(axes), initial_value, **kw)


def constant(const, axes=None, dtype=None, **kw):
    const = np.asarray(const, dtype=np.float32)
    if axes is None:
        if const.ndim:
            raise ValueError("a non-scalar constant needs axes")
        axes = ()
    return AssignableTensorOp(make_axes(axes), const, is_constant=True, is_persistent=True, **kw)


def as_op(x):
    if isinstance(x, Op):
        return x
    if isinstance(x, (numbers.Number, np.number, np.bool_)) or \
            (isinstance(x, np.ndarray) and x.ndim == 0):
        return constant(float(x))
    raise ValueError("cannot use %r as a graph op" % (x,))


def as_ops(xs):
    return tuple(as_op(x) for x in xs)


# ---- views ----------------------------------------------------------------------------------
class ViewOp(Op):
    """Ops that re-describe their argument's storage without moving data (the reference's
    IndexOp family, ngraph/op_graph/op_graph.py:1650-1715)."""
    is_device_op = False


class BroadcastOp(ViewOp):
    def __init__(self, x, axes, **kw):
        x = as_op(x)
        axes = make_axes(axes)
        if not x.axes.is_sub_set(axes):
            raise ValueError("The new axes %s are not a superset of the op's axes %s" %
                             (axes, x.axes))
        super(BroadcastOp, self).__init__((x,), axes, **kw)


class ReorderAxes(ViewOp):
    def __init__(self, x, axes, **kw):
        x = as_op(x)
        axes = make_axes(axes)
        if not x.axes.is_equal_set(axes):
            raise ValueError("The input axes %s and output axes %s must have the same members" %
                             (x.axes, axes))
        super(ReorderAxes, self).__init__((x,), axes, **kw)


class AxesCastOp(ViewOp):
    """Same storage, new axes position by position (ngraph/op_graph/op_graph.py: AxesCastOp)."""

    def __init__(self, x, axes, **kw):
        x = as_op(x)
        axes = make_axes(axes)
        if x.axes.lengths != axes.lengths:
            raise ValueError("casting axes {} must have the same length as original axes {}"
                             .format(axes, x.axes))
        super(AxesCastOp, self).__init__((x,), axes, **kw)


class ReshapeOp(ViewOp):
    """The same elements in the same order under other axes: neighbouring axes merged into one or
    one axis split into several (the reference's Flatten / Unflatten,
    ngraph/op_graph/op_graph.py:2221-2294, whose FlattenedAxis has the product of its members'
    lengths).  No data moves; the argument's storage must allow it (a dense tensor always does)."""

    def __init__(self, x, axes, **kw):
        x = as_op(x)
        axes = make_axes(axes)
        if x.axes.size != axes.size:
            raise ValueError("reshape from {} to {} changes the number of elements"
                             .format(x.axes, axes))
        super(ReshapeOp, self).__init__((x,), axes, **kw)


def reshape(x, axes):
    x = as_op(x)
    axes = make_axes(axes)
    if x.axes == axes:
        return x
    return ReshapeOp(x, axes)


class TensorSliceOp(ViewOp):
    """A sliced view: one slice or int per axis of x; an int drops the axis
    (ngraph/op_graph/op_graph.py:2067-2120).  Negative steps are not supported, as there."""

    def __init__(self, x, slices, axes=None, **kw):
        x = as_op(x)
        slices = tuple(slices)
        if len(slices) != len(x.axes):
            raise ValueError("There should be one slice in slices for each dimension in input "
                             "tensor.  Input tensor had {} dimensions, but slices has length {}."
                             .format(len(x.axes), len(slices)))
        kept, starts, steps = [], [], []
        for axis, sl in zip(x.axes, slices):
            if isinstance(sl, slice):
                if sl.step is not None and sl.step < 0:
                    raise ValueError("Negative slice steps are not supported.")
                start, stop, step = sl.indices(axis.length)
                n = -(-(stop - start) // step)        # (max / min are reductions in this module)
                n = n if n > 0 else 0
                kept.append(axis if (start, n, step) == (0, axis.length, 1)
                            else make_axis(n, name=axis.name))
                starts.append(start)
                steps.append(step)
            else:
                idx = int(sl)
                if idx < 0:
                    idx += axis.length
                if not 0 <= idx < axis.length:
                    raise ValueError("index %d is out of range for axis %s" % (int(sl), axis))
                starts.append(idx)
                steps.append(None)          # the axis is dropped
        if axes is None:
            axes = kept
        axes = make_axes(axes)
        if axes.lengths != make_axes(kept).lengths:
            raise ValueError("slice result has shape %s, the given axes %s"
                             % (make_axes(kept).lengths, axes.lengths))
        super(TensorSliceOp, self).__init__((x,), axes, **kw)
        self.slices = slices
        self.starts = tuple(starts)
        self.steps = tuple(steps)


def tensor_slice(x, slices, axes=None):
    return TensorSliceOp(x, slices, axes)


def cast_axes(tensor, axes):
    tensor = as_op(tensor)
    axes = make_axes(axes)
    if tensor.axes == axes:
        return tensor
    return AxesCastOp(tensor, axes)


def broadcast(x, axes):
    x = as_op(x)
    axes = make_axes(axes)
    if x.axes == axes:
        return x
    return BroadcastOp(x, axes)


def axes_with_order(x, axes):
    x = as_op(x)
    axes = make_axes(axes)
    if x.axes == axes:
        return x
    return ReorderAxes(x, axes)


# ---- elementwise ------------------------------------------------------------------------------
class ElementWiseOp(Op):
    def __init__(self, opname, args, **kw):
        args = as_ops(args)
        axes = Axes()
        for a in args:
            axes = axes + a.axes
        super(ElementWiseOp, self).__init__(args, axes, **kw)
        self.opname = opname


def _unary(opname):
    def build(x, **kw):
        return ElementWiseOp(opname, (x,), **kw)
    build.__name__ = opname
    return build


def _binary(opname):
    def build(x, y, dtype=None, **kw):
        return ElementWiseOp(opname, (x, y), **kw)
    build.__name__ = opname
    return build


negative = _unary("neg")
absolute = _unary("abs")
sin = _unary("sin")
cos = _unary("cos")
tanh = _unary("tanh")
exp = _unary("exp")
log = _unary("log")
reciprocal = _unary("rcp")
sign = _unary("sgn")
square = _unary("sqr")
sqrt = _unary("sqrt")
sigmoidAtomic = _unary("sig")

add = _binary("add")
subtract = _binary("sub")
multiply = _binary("mul")
divide = _binary("div")
floordivide = _binary("int_div")
mod = _binary("mod")
maximum = _binary("maximum")
minimum = _binary("minimum")
power = _binary("pow")
equal = _binary("eq")
not_equal = _binary("ne")
greater = _binary("gt")
less = _binary("lt")
greater_equal = _binary("ge")
less_equal = _binary("le")


safelog_cutoff = 50.0


def safelog(x, limit=-safelog_cutoff):
    """maximum(log(x + exp(limit)), limit) (ngraph/op_graph/op_graph.py:3067-3072)."""
    return maximum(log(x + float(np.exp(limit))), limit)


def sigmoid(x):
    """reciprocal(exp(-x) + 1), as the reference composes it
    (ngraph/op_graph/op_graph.py:4183-4199)."""
    return reciprocal(exp(negative(x)) + 1)


# ---- reductions -------------------------------------------------------------------------------
def compute_reduction_axes(x, reduction_axes, out_axes):
    """ngraph/op_graph/op_graph.py: compute_reduction_axes."""
    if reduction_axes is None and out_axes is None:
        reduction_axes = x.axes - x.axes.find_by_name("N")   # sample axes
        out_axes = x.axes - reduction_axes
    elif reduction_axes is None:
        out_axes = make_axes(out_axes)
        reduction_axes = x.axes - out_axes
    elif out_axes is None:
        reduction_axes = make_axes(reduction_axes)
        out_axes = x.axes - reduction_axes
    else:
        out_axes = make_axes(out_axes)
        reduction_axes = make_axes(reduction_axes)
    if not reduction_axes.is_sub_set(x.axes):
        raise ValueError("reduction axes %s are not axes of the operand %s" %
                         (reduction_axes, x.axes))
    return reduction_axes, out_axes


class ReductionOp(Op):
    def __init__(self, redop, x, reduction_axes=None, out_axes=None, **kw):
        x = as_op(x)
        reduction_axes, out_axes = compute_reduction_axes(x, reduction_axes, out_axes)
        super(ReductionOp, self).__init__((x,), out_axes, **kw)
        self.redop = redop
        self.reduction_axes = reduction_axes


def _reduction(redop):
    def build(x, reduction_axes=None, out_axes=None, dtype=None, **kw):
        return ReductionOp(redop, x, reduction_axes, out_axes, **kw)
    build.__name__ = redop
    return build


sum = _reduction("sum")          # noqa: A001  (the reference shadows the builtins the same way)
prod = _reduction("prod")
max = _reduction("max")          # noqa: A001
min = _reduction("min")          # noqa: A001
argmax = _reduction("argmax")
argmin = _reduction("argmin")


def mean(x, reduction_axes=None, out_axes=None):
    """ngraph/op_graph/op_graph.py:4252-4266."""
    x = as_op(x)
    reduction_axes, out_axes = compute_reduction_axes(x, reduction_axes, out_axes)
    return sum(x, reduction_axes=reduction_axes, out_axes=out_axes) / float(reduction_axes.size)


def variance(x, out_axes=None, reduction_axes=None):
    """ngraph/op_graph/op_graph.py:4007-4009: mean of the squared distance from the mean."""
    x = as_op(x)
    return mean(square(x - mean(x, reduction_axes=reduction_axes, out_axes=out_axes)),
                reduction_axes=reduction_axes, out_axes=out_axes)


def softmax(x, normalization_axes=None, **kw):
    """ngraph/op_graph/op_graph.py: SoftmaxOp -- exp(x - max) / sum(exp(x - max))."""
    x = as_op(x)
    if normalization_axes is None:
        normalization_axes = x.axes - x.axes.find_by_name("N")
    normalization_axes = make_axes(normalization_axes)
    e = exp(x - max(x, reduction_axes=normalization_axes))
    return e * reciprocal(sum(e, reduction_axes=normalization_axes))


# ---- contractions -------------------------------------------------------------------------------
class DotOp(Op):
    """Contracts the axes common to both operands (ngraph/op_graph/op_graph.py: DotOp)."""

    def __init__(self, x, y, **kw):
        x, y = as_op(x), as_op(y)
        self.reduction_axes = x.axes & y.axes
        self.x_out_axes = x.axes - self.reduction_axes
        self.y_out_axes = y.axes - self.reduction_axes
        super(DotOp, self).__init__((x, y), self.x_out_axes + self.y_out_axes, **kw)


def dot(x, y):
    return DotOp(x, y)


class ConvolutionOp(Op):
    """fprop: O[K,M,P,Q,N] = sum F[C,T,R,S,K] * I[C,D,H,W,N]
    (ngraph/op_graph/convolution.py:  ConvolutionOp)."""

    def __init__(self, conv_params, inputs, filters, axes, bias=None, activation=None,
                 residual=None, **kw):
        inputs, filters = as_op(inputs), as_op(filters)
        if len(inputs.axes) != 5:
            raise ValueError("convolution input shape must be length 5, found {}".format(
                len(inputs.axes.lengths)))
        if len(filters.axes) != 5:
            raise ValueError("convolution filter shape must be length 5, found {}".format(
                len(filters.axes.lengths)))
        if inputs.axes[0].length != filters.axes[0].length:
            raise ValueError("the first axis in input {inputs} and filter {filters} are not the "
                             "same.".format(inputs=inputs.axes[0], filters=filters.axes[0]))
        args = [inputs, filters]
        super(ConvolutionOp, self).__init__(args, axes, **kw)
        self.conv_params = dict(conv_params)


def convolution(conv_params, inputs, filters, axes, **kw):
    return ConvolutionOp(conv_params, inputs, filters, make_axes(axes), **kw)


class ConvDerivOp(Op):
    """Common part of the two convolution gradients: they carry the forward op, whose
    conv_params and tensor extents they share (ngraph/op_graph/convolution.py: ConvDerivOp)."""

    def __init__(self, args, fprop, axes, **kw):
        if not isinstance(fprop, ConvolutionOp):
            raise ValueError("fprop must be the forward ConvolutionOp")
        super(ConvDerivOp, self).__init__(args, axes, **kw)
        self.fprop = fprop
        self.conv_params = fprop.conv_params
        self.add_control_dep(fprop)


class update_conv(ConvDerivOp):
    """Filter gradient U[C,T,R,S,K] = sum_{p,q,n} I * delta
    (ngraph/op_graph/convolution.py: update_conv; args are (delta, inputs))."""

    def __init__(self, delta, inputs, filters, fprop, **kw):
        delta, inputs = as_op(delta), as_op(inputs)
        super(update_conv, self).__init__((delta, inputs), fprop, as_op(filters).axes, **kw)


class bprop_conv(ConvDerivOp):
    """Input gradient gI[C,D,H,W,N] = sum_{k,r,s} F * delta
    (ngraph/op_graph/convolution.py: bprop_conv; args are (delta, filters))."""

    def __init__(self, delta, inputs, filters, fprop, **kw):
        delta, filters = as_op(delta), as_op(filters)
        super(bprop_conv, self).__init__((delta, filters), fprop, as_op(inputs).axes, **kw)


class PoolingOp(Op):
    """ngraph/op_graph/pooling.py: PoolingOp; input C,D,H,W,N -> output C,M,P,Q,N."""

    def __init__(self, pool_params, inputs, axes, **kw):
        inputs = as_op(inputs)
        if len(inputs.axes) != 5:
            raise ValueError("pooling input shape must be length 5, found {}".format(
                len(inputs.axes.lengths)))
        if pool_params["op"] not in ("max", "avg"):
            raise ValueError("Unsupported pooling type: {pooltype}.  Only max and avg pooling "
                             "currently supported. ".format(pooltype=pool_params["op"]))
        super(PoolingOp, self).__init__((inputs,), axes, **kw)
        self.pool_params = dict(pool_params)


def pooling(pool_params, inputs, axes, **kw):
    return PoolingOp(pool_params, inputs, make_axes(axes), **kw)


class BpropPoolOp(Op):
    """Gradient of a PoolingOp with respect to its input (ngraph/op_graph/pooling.py:70-93):
    args (delta C,M,P,Q,N ; the pooled tensor C,D,H,W,N), result on the pooled tensor's axes."""

    def __init__(self, delta, inputs, fprop, **kw):
        delta, inputs = as_op(delta), as_op(inputs)
        if not isinstance(fprop, PoolingOp):
            raise ValueError("bprop_pool needs the forward PoolingOp, got {}".format(fprop))
        if delta.axes.lengths != fprop.axes.lengths:
            raise ValueError("bprop_pool: delta has shape %s, the pooling result %s"
                             % (delta.axes.lengths, fprop.axes.lengths))
        super(BpropPoolOp, self).__init__((delta, inputs), inputs.axes, **kw)
        self.fprop = fprop

    @property
    def pool_params(self):
        return self.fprop.pool_params


def bprop_pool(delta, inputs, fprop):
    return BpropPoolOp(delta, inputs, fprop)


class LookupTableOp(Op):
    """out = lut.take(idx, axis) (ngraph/op_graph/lookuptable.py:55-118): lut is 2-d, idx 1-d;
    the output axes name the index axis in place of the lut axis that is looked up."""

    def __init__(self, lut, idx, axes, update=True, pad_idx=None, **kw):
        lut, idx = as_op(lut), as_op(idx)
        axes = make_axes(axes)
        if len(lut.axes) != 2:
            raise ValueError("lookup table shape must be length 2, found {}".format(len(lut.axes)))
        if len(idx.axes) != 1:
            raise ValueError("index shape must be length 1, found {}".format(len(idx.axes)))
        if not (lut.axes[0] in axes or lut.axes[1] in axes):
            raise ValueError("Output axes must indicate which axis to do lookup.  None of the "
                             "output axes is from lookup table.")
        if idx.axes[0] not in axes:
            raise ValueError("Output axes must index axes.")
        self.lut_axis = 0 if lut.axes[1] in axes else 1
        self.pad_idx = pad_idx
        self.update = update
        if axes[self.lut_axis] != idx.axes[0]:
            raise ValueError("Cannot transpose lut axes implicitly")
        super(LookupTableOp, self).__init__((lut, idx), axes, **kw)


def lookuptable(lut, idx, axes, update=True, pad_idx=None, **kw):
    return LookupTableOp(lut, idx, axes, update=True, pad_idx=pad_idx)


class update_lut(Op):    # noqa: N801  (the reference's name)
    """Gradient of the table: args (delta, idx), result on the table's axes
    (ngraph/op_graph/lookuptable.py:160-175)."""

    def __init__(self, delta, lut, idx, fprop, **kw):
        delta, lut, idx = as_op(delta), as_op(lut), as_op(idx)
        if not isinstance(fprop, LookupTableOp):
            raise ValueError("update_lut needs the forward LookupTableOp, got {}".format(fprop))
        if delta.axes.lengths != fprop.axes.lengths:
            raise ValueError("update_lut: delta has shape %s, the lookup result %s"
                             % (delta.axes.lengths, fprop.axes.lengths))
        super(update_lut, self).__init__((delta, idx), lut.axes, **kw)
        self.fprop = fprop

    @property
    def lut_axis(self):
        return self.fprop.lut_axis

    @property
    def pad_idx(self):
        return self.fprop.pad_idx


def lookuptable_update(delta, lut, idx, fprop_op):
    return update_lut(delta, lut, idx, fprop_op)


# ---- communication ----------------------------------------------------------------------------
class AllReduceOp(Op):
    """Sum (or mean) of a tensor over all data-parallel replicas; every replica gets the result
    (ngraph/op_graph/comm_nodes.py:347-383 GPUCudaAllReduceOp; inserted by hetr wherever an
    argument carries reduce_func and its consumer does not,
    ngraph/factory/comm_node_factory.py:298-341)."""

    def __init__(self, x, reduce_func="sum", **kw):
        x = as_op(x)
        if reduce_func not in ("sum", "mean"):
            raise ValueError("unsupported reduce_func %r" % (reduce_func,))
        super(AllReduceOp, self).__init__((x,), x.axes, **kw)
        self.reduce_func = reduce_func


class RngOp(Op):
    """A tensor with the axes of x, filled with fresh random numbers on every execution
    (ngraph/op_graph/op_graph.py:2786-2870; x only supplies the axes, as in the reference's
    kernels, ngraph/transformers/gpu/tensor_ops.py:621-661)."""

    def __init__(self, distribution, params, x, **kw):
        if distribution not in ("uniform", "normal"):
            raise ValueError("unsupported distribution: {}".format(distribution))
        x = as_op(x)
        self.distribution = distribution
        self.params = dict(params)
        super(RngOp, self).__init__((x,), x.axes, **kw)


def uniform(x, low=0.0, high=1.0):
    return RngOp("uniform", dict(low=low, high=high), x)


def normal(x, loc=0.0, scale=1.0):
    return RngOp("normal", dict(loc=loc, scale=scale), x)


def allreduce(x, reduce_func="sum"):
    return AllReduceOp(x, reduce_func)


# ---- state and control ------------------------------------------------------------------------
class AssignOp(Op):
    """tensor <- value (ngraph/op_graph/op_graph.py: AssignOp)."""
    is_tensor_op = False

    def __init__(self, tensor, val, **kw):
        tensor, val = as_op(tensor), as_op(val)
        base = tensor
        while isinstance(base, ViewOp):              # a view of an assignable tensor is assignable
            base = base.args[0]
        if not isinstance(base, AssignableTensorOp):
            raise ValueError("{} is not assignable.".format(tensor))
        if not val.axes.is_sub_set(tensor.axes):
            raise ValueError("cannot assign axes %s to a tensor with axes %s" %
                             (val.axes, tensor.axes))
        super(AssignOp, self).__init__((tensor, val), tensor.axes, **kw)


def assign(lvalue, rvalue):
    return AssignOp(lvalue, rvalue)


class SequentialOp(Op):
    """Runs `ops` in order; its value is the last one (ngraph/op_graph/op_graph.py:
    SequentialOp)."""
    is_device_op = False

    def __init__(self, ops, **kw):
        ops = as_ops(ops)
        if not ops:
            raise ValueError("sequential needs at least one op")
        super(SequentialOp, self).__init__(ops, ops[-1].axes, **kw)
        self.ops = ops

    @property
    def value_tensor(self):
        return self.ops[-1]


def sequential(ops=None):
    return SequentialOp(ops)


def value_of(tensor):
    """A copy of the tensor's current value (ngraph/op_graph/op_graph.py: value_of)."""
    return ElementWiseOp("assign", (tensor,))
