"""Plug-in that registers the b200 transformer INSIDE an nGraph-Python installation.

    import ngraph_python_b200.ngraph_plugin          # registers transformer_name = 'b200'
    import ngraph.transformers as ngt
    t = ngt.make_transformer_factory('b200', flex=True)()
    f = t.computation(outputs, *placeholders)         # ordinary ngraph ops
    y = f(x)

The reference registers every `Transformer` subclass that defines `transformer_name`
(ngraph/transformers/base.py:265-279) and reaches it through make_transformer_factory /
allocate_transformer (:834-847).  This class takes a ComputationOp (what
`Transformer.computation` builds, base.py:420-433, op_graph.py:961-1033), translates the graph it
returns into the op surface of this package (same op names and argument meaning, so the mapping
is one line per op class) and hands it to the b200 planner.  The reference's own graph passes,
CPU code generator and GPU back end are not involved.

Only importable where `ngraph` itself imports.
"""
import collections
import os

import numpy as np

import ngraph.op_graph.op_graph as ref
from ngraph.op_graph.convolution import ConvolutionOp as RefConvolutionOp
from ngraph.op_graph.convolution import bprop_conv as ref_bprop_conv
from ngraph.op_graph.convolution import update_conv as ref_update_conv
from ngraph.op_graph.convolution import DeconvolutionOp as RefDeconvolutionOp
from ngraph.op_graph.convolution import DeconvDerivOp as RefDeconvDerivOp
from ngraph.op_graph.pooling import PoolingOp as RefPoolingOp, BpropPoolOp as RefBpropPoolOp
from ngraph.op_graph.lookuptable import LookupTableOp as RefLookupTableOp, update_lut as ref_update_lut
from ngraph.transformers.base import Transformer

from . import op_graph as b2
from . import transformers as b2t

_UNARY = {
    "NegativeOp": b2.negative, "AbsoluteOp": b2.absolute, "SinOp": b2.sin, "CosOp": b2.cos,
    "TanhOp": b2.tanh, "ExpOp": b2.exp, "LogOp": b2.log, "ReciprocalOp": b2.reciprocal,
    "SignOp": b2.sign, "SquareOp": b2.square, "SqrtOp": b2.sqrt,
    "SigmoidAtomicOp": b2.sigmoidAtomic,
}
_BINARY = {
    "Add": b2.add, "Subtract": b2.subtract, "Multiply": b2.multiply, "Divide": b2.divide,
    "FloorDivide": b2.floordivide, "Mod": b2.mod, "Maximum": b2.maximum, "Minimum": b2.minimum,
    "Power": b2.power, "Equal": b2.equal, "NotEqual": b2.not_equal, "Greater": b2.greater,
    "Less": b2.less, "GreaterEqual": b2.greater_equal, "LessEqual": b2.less_equal,
}
_REDUCE = {"Sum": b2.sum, "Prod": b2.prod, "Max": b2.max, "Min": b2.min, "Argmax": b2.argmax,
           "Argmin": b2.argmin}


def _is_zero(op):
    """A scalar constant 0 of the mirror graph (possibly broadcast)."""
    while isinstance(op, b2.ViewOp):
        op = op.args[0]
    return (isinstance(op, b2.AssignableTensorOp) and getattr(op, "is_scalar_constant", False) and
            float(np.asarray(op.initial_value)) == 0.0)


def _reduce_tag(op):
    """The reduce_func an op is tagged with (a ValueOp carries the tag of its value tensor)."""
    op = op.forwarded
    while True:
        rf = op.metadata.get("reduce_func")
        if rf:
            return rf
        if isinstance(op, ref.ValueOp):
            op = op.value_tensor.forwarded
            continue
        return None


def _find_parallel_axis(computation_op):
    """The axis named by `parallel=` in the metadata of the graph's ops (hetr's device
    annotation: `with ng.metadata(device='gpu', device_id=('0', '1'), parallel=ax.N)`), or None."""
    seen, stack = set(), [computation_op]
    while stack:
        op = stack.pop()
        if op in seen:
            continue
        seen.add(op)
        axis = op.metadata.get("parallel") if hasattr(op, "metadata") else None
        if axis is not None:
            return axis
        stack.extend(op.all_deps)
        if isinstance(op, ref.ValueOp):
            stack.append(op.value_tensor)
    return None


class GraphTranslator(object):
    """reference Op -> ngraph_python_b200 Op, memoised.

    replicas > 1: the graph is one replica's share of a data-parallel job.  An exchange is placed
    wherever the reference's communication pass would place one: between a tensor tagged with
    `reduce_func` -- autodiff tags every gradient 'sum' (ngraph/op_graph/op_graph.py:4294-4297)
    -- and a consumer without the tag (ngraph/factory/comm_node_factory.py:314-318,
    ngraph/transformers/passes/hetrpasses.py:63-89).  shard_batch: every replica built its graph
    on its own shard of the global batch, so the optimizer's `/ batch_size`
    (ngraph/frontends/neon/optimizer.py:177-198) divides by the shard's size; the summed gradient
    is then also divided by the number of replicas, which makes it the division by the global
    batch size the reference performs."""

    def __init__(self, replicas=1, shard_batch=True, parallel_axis=None, rank=0):
        self.memo = {}
        self.bare = {}       # AssignableTensorOp -> its translation (shared with memo)
        self.axis_memo = {}
        self.replicas = int(replicas)
        self.shard_batch = bool(shard_batch)
        self.exchanges = {}  # tagged reference op -> its allreduce
        # hetr-style graphs: built on the GLOBAL batch under ng.metadata(device_id=(...),
        # parallel=axis); every replica runs the same graph with that axis cut to its share
        # (what hetr's DeviceAssignPass / scatter does, ngraph/transformers/passes/hetrpasses.py:
        # 98-131, ngraph/op_graph/comm_nodes.py:180-215)
        self.parallel_axis = parallel_axis
        self.rank = int(rank)

    def set_parallel_axis(self, axis):
        if axis is None or self.replicas <= 1:
            return
        if self.parallel_axis is not None and (self.parallel_axis.name != axis.name or
                                               self.parallel_axis.length != axis.length):
            raise ValueError("computations of one transformer must agree on the parallel axis")
        if axis.length % self.replicas:
            raise ValueError("the parallel axis {} does not divide over {} replicas"
                             .format(axis, self.replicas))
        if self.parallel_axis is None and self.axis_memo:
            raise ValueError("the parallel axis must be known before the first translation")
        self.parallel_axis = axis
        self.shard_batch = False     # the graph's batch size is the global one already

    def is_parallel(self, a):
        p = self.parallel_axis
        return p is not None and a.name == p.name and a.length == p.length

    def axis(self, a):
        if getattr(a, "is_flattened", False):
            # a FlattenedAxis is what it is made of: two of them over the same axes are the same
            # axis (the reference compares them by their members, not by their generated names)
            name = "flat(" + ",".join(self.axis(m).name for m in a.axes) + ")"
        else:
            name = a.name
        length = a.length // self.replicas if self.is_parallel(a) else a.length
        key = (name, a.length)
        if key not in self.axis_memo:
            self.axis_memo[key] = b2.make_axis(length, name=name)
        return self.axis_memo[key]

    def axes(self, axes):
        return b2.make_axes([self.axis(a) for a in axes])

    def __call__(self, op):
        op = op.forwarded
        if op in self.memo:
            return self.memo[op]
        out = self.bare[op] if op in self.bare else self._translate(op)
        if isinstance(op, ref.AssignableTensorOp):
            self.bare[op] = out
        # Order is part of the contract (Op.ordered_ops sorts over args and control_deps): an op
        # that must run after others -- a TensorValueOp reading a tensor after the assignments
        # that build it, as the adjoint of a slice does -- becomes the last op of a sequential.
        deps = [d.forwarded for d in getattr(op, "control_deps", ())]
        if deps and not isinstance(op, ref.ParallelOp):
            out = b2.sequential([self(d) for d in deps] + [out])
        self.memo[op] = out
        return out

    def _arg(self, consumer, a):
        """Translation of argument `a` as `consumer` reads it: through an allreduce where the
        reference's communication pass would put one."""
        if self.replicas > 1 and "reduce_func" not in consumer.metadata:
            rf = _reduce_tag(a)
            if rf is not None:
                key = a.forwarded
                if key not in self.exchanges:
                    func = "mean" if (rf == "sum" and self.shard_batch) else rf
                    self.exchanges[key] = b2.allreduce(self(a), reduce_func=func)
                return self.exchanges[key]
        return self(a)

    def _target(self, op):
        """(translated assignment target without sequencing wrappers, ops that must run first)."""
        op = op.forwarded
        before = [self(d.forwarded) for d in getattr(op, "control_deps", ())]
        if isinstance(op, ref.ValueOp):
            t, b = self._target(op.value_tensor)
            return t, before + b
        if isinstance(op, ref.TensorSliceOp):
            t, b = self._target(op.args[0])
            return b2.tensor_slice(t, op.slices, self.axes(op.axes)), before + b
        if isinstance(op, ref.AxesCastOp):
            t, b = self._target(op.args[0])
            return b2.cast_axes(t, self.axes(op.axes)), before + b
        if isinstance(op, ref.AssignableTensorOp):
            if op not in self.bare:
                self.bare[op] = self._translate(op)
            return self.bare[op], before
        raise ValueError("Unhandled op: assignment to {}".format(op))

    def _translate(self, op):
        name = type(op).__name__
        if isinstance(op, ref.AssignableTensorOp):
            init = op.initial_value
            if op.is_constant and init is None:
                init = op.const
            kw = dict(is_input=op.is_input, is_persistent=op.is_persistent,
                      is_constant=op.is_constant, is_trainable=op.is_trainable,
                      is_placeholder=op.is_placeholder, name=op.name)
            if init is not None and not callable(init):
                init = np.asarray(init, dtype=np.float32)
                for pos, a in enumerate(op.axes):
                    # a tensor initialised along the parallel axis: this replica's share of it
                    if self.is_parallel(a) and init.ndim == len(op.axes) and \
                            init.shape[pos] == a.length:
                        share = a.length // self.replicas
                        init = np.take(init, range(self.rank * share, (self.rank + 1) * share),
                                       axis=pos)
            return b2.AssignableTensorOp(self.axes(op.axes), init, **kw)
        if isinstance(op, ref.SequentialOp):
            return b2.sequential([self(o) for o in op.ops])
        if isinstance(op, ref.ParallelOp):              # doall: any order will do; keep the given one
            return b2.sequential([self(o) for o in op.control_deps])
        if isinstance(op, ref.ValueOp):                 # sigmoid, softmax, mean, ... expand
            return self(op.value_tensor)
        if isinstance(op, ref.AssignOp):
            # the target is the tensor (or a view of it) itself; what its description must run
            # after (a Fill of the same tensor, say) runs before the assignment
            target, before = self._target(op.args[0])
            assign = b2.assign(target, self._arg(op, op.args[1]))
            return b2.sequential(before + [assign]) if before else assign
        if isinstance(op, ref.Fill):
            return b2.assign(self(op.args[0]), b2.constant(float(op.scalar)))
        if isinstance(op, ref.TensorSizeOp):
            # the number of elements along the reduction axes (what mean and variance divide by:
            # ngraph/op_graph/op_graph.py:4012-4029); the reference folds it into a constant too
            return b2.constant(float(op.reduction_axes.size))
        args = [self._arg(op, a) for a in op.args]
        if name in _UNARY:
            return _UNARY[name](args[0])
        if name in _BINARY:
            # The reference's Rectlin is maximum(x, 0) + slope * minimum(x, 0) with slope 0 for a
            # plain ReLU; its SimplePrune pass folds the dead half away
            # (ngraph/transformers/passes/passes.py), and so does this translation.
            if name == "Multiply" and (_is_zero(args[0]) or _is_zero(args[1])):
                zero = b2.constant(0.0)
                return b2.broadcast(zero, self.axes(op.axes)) if len(op.axes) else zero
            if name == "Add" and _is_zero(args[1]) and args[0].axes == self.axes(op.axes):
                return args[0]
            if name == "Add" and _is_zero(args[0]) and args[1].axes == self.axes(op.axes):
                return args[1]
            return _BINARY[name](args[0], args[1])
        if name in _REDUCE:
            return _REDUCE[name](args[0], reduction_axes=self.axes(op.reduction_axes))
        if isinstance(op, ref.DotOp):
            return b2.dot(args[0], args[1])
        if isinstance(op, ref.BroadcastOp):
            return b2.broadcast(args[0], self.axes(op.axes))
        if isinstance(op, ref.ReorderAxes):
            return b2.axes_with_order(args[0], self.axes(op.axes))
        if isinstance(op, ref.OneHotOp):
            # (class axis) + x.axes; element = 1 where the class index equals x
            classes = self.axes([op.axis])
            iota = b2.constant(np.arange(classes[0].length, dtype=np.float32), axes=classes)
            return b2.equal(iota, args[0])
        if isinstance(op, ref.TensorSliceOp):
            return b2.tensor_slice(args[0], op.slices, self.axes(op.axes))
        if isinstance(op, ref.AxesCastOp):
            return b2.cast_axes(args[0], self.axes(op.axes))
        if isinstance(op, ref.ExpandDims):
            return b2.broadcast(args[0], self.axes(op.axes))
        if isinstance(op, RefConvolutionOp):
            return b2.convolution(dict(op.conv_params), args[0], args[1], self.axes(op.axes))
        if isinstance(op, RefDeconvolutionOp):
            # A deconvolution is the input gradient of the convolution that would take its result
            # back to its argument (the reference runs it on its ConvBpropKernel the same way,
            # ngraph/transformers/gputransform.py: DeconvolutionOp).  That convolution exists
            # here only as the carrier of the dimensions.
            shape_of_result = b2.temporary(self.axes(op.axes))
            carrier = b2.convolution(dict(op.conv_params), shape_of_result, args[1],
                                     self.axes(op.args[0].axes))
            return b2.bprop_conv(args[0], shape_of_result, args[1], carrier)
        if isinstance(op, RefDeconvDerivOp):         # args (delta, filters): a forward convolution
            fprop = self(op.fprop)
            carrier = fprop.fprop if isinstance(fprop, b2.bprop_conv) else fprop
            return b2.convolution(dict(carrier.conv_params), args[0], args[1], self.axes(op.axes))
        if isinstance(op, ref_bprop_conv):           # args (delta, filters)
            fprop = self(op.fprop)
            return b2.bprop_conv(args[0], fprop.args[0], args[1], fprop)
        if isinstance(op, ref_update_conv):          # args (delta, inputs)
            fprop = self(op.fprop)
            if isinstance(fprop, b2.bprop_conv):     # gradient of a deconvolution's filters
                fprop = fprop.fprop
            return b2.update_conv(args[0], args[1], fprop.args[1], fprop)
        if isinstance(op, RefPoolingOp):
            return b2.pooling(dict(op.pool_params), args[0], self.axes(op.axes))
        if isinstance(op, RefBpropPoolOp):            # args (delta,); the pooled tensor via fprop
            fprop = self(op.fprop)
            return b2.bprop_pool(args[0], fprop.args[0], fprop)
        if isinstance(op, RefLookupTableOp):
            return b2.lookuptable(args[0], args[1], self.axes(op.axes), pad_idx=op.pad_idx)
        if isinstance(op, ref_update_lut):            # args (delta, idx); the table via fprop
            fprop = self(op.fprop)
            return b2.update_lut(args[0], fprop.args[0], args[1], fprop)
        if isinstance(op, (ref.Flatten, ref.Unflatten)):
            return b2.reshape(args[0], self.axes(op.axes))
        if isinstance(op, ref.RngOp):
            return b2.RngOp(op.distribution, op.params, args[0])
        if isinstance(op, ref.ContiguousOp):
            # a freshly computed tensor is dense already; views and variables are copied
            if isinstance(args[0], (b2.ViewOp, b2.AssignableTensorOp, b2.SequentialOp)):
                return b2.value_of(args[0])
            return args[0]
        raise ValueError("Unhandled op: {}".format(op))


class _PluginComputation(object):
    """Callable with the calling conventions of ngraph.transformers.base.Computation
    (base.py:73-136): positional arguments or feed_dict; scalar / tuple / dict results."""

    def __init__(self, transformer, computation_op):
        self.transformer = transformer
        self.computation_op = computation_op
        tr = transformer.translator
        returns = computation_op.returns
        if tr.replicas > 1:
            tr.set_parallel_axis(_find_parallel_axis(computation_op))
        self.dict_keys = None
        if isinstance(returns, dict):
            self.dict_keys = list(returns.keys())
            outs = [tr(returns[k]) for k in self.dict_keys]
        elif isinstance(returns, collections.abc.Set) and not isinstance(returns, ref.Op) and \
                type(returns).__name__ != "OrderedSet":
            # an unordered set of ops comes back as a dict keyed by op (base.py:128-132)
            self.dict_keys = list(returns)
            outs = [tr(r) for r in self.dict_keys]
        elif isinstance(returns, collections.abc.Container) and not isinstance(returns, ref.Op):
            outs = [tr(r) for r in returns]
        elif returns is None:
            outs = None
        else:
            outs = tr(returns)
        self.parameters = list(computation_op.parameters)
        params = [tr(p.tensor) for p in self.parameters]
        self.impl = transformer.impl.computation(outs, *params)
        self.returns = returns
        # position of the parallel axis in every parameter that has it: the caller passes the
        # global array, this replica takes its slice (hetr's scatter)
        self.scatter = [next((i for i, a in enumerate(p.tensor.axes) if tr.is_parallel(a)), None)
                        for p in self.parameters]

    def capture(self):
        """Replays the computation as one CUDA graph from now on (call it after a first run)."""
        self.impl.capture()
        return self

    def _gather(self, res):
        """Results that carry the parallel axis, put together from all replicas along it."""
        tr = self.transformer.translator
        comm = self.transformer.impl.comm
        ops = _result_ops(self.returns)
        single = isinstance(self.returns, ref.Op)
        vals = [res] if single else list(res)
        out = []
        for op, v in zip(ops, vals):
            pos = next((i for i, a in enumerate(op.axes) if tr.is_parallel(a)), None)
            out.append(v if pos is None else comm.all_gather_host(np.asarray(v), pos))
        return out[0] if single else tuple(out)

    def __call__(self, *args, **kwargs):
        feed = kwargs.pop("feed_dict", None)
        if feed is not None:
            args = [feed[p.tensor] if p.tensor in feed else feed[p] for p in self.parameters]
        tr = self.transformer.translator
        if tr.parallel_axis is not None:
            rank, n = self.transformer.impl.comm.rank, tr.replicas
            cut = []
            for a, pos in zip(args, self.scatter):
                if pos is not None and np.ndim(a) > pos and np.shape(a)[pos] == tr.parallel_axis.length:
                    share = np.shape(a)[pos] // n
                    index = [slice(None)] * np.ndim(a)
                    index[pos] = slice(rank * share, (rank + 1) * share)
                    a = np.ascontiguousarray(np.asarray(a)[tuple(index)])
                cut.append(a)
            args = cut
        res = self.impl(*args)
        if tr.parallel_axis is not None and self.transformer.gather_results:
            res = self._gather(res)
        if self.dict_keys is not None:
            return dict(zip(self.dict_keys, res))
        if isinstance(self.returns, ref.Op) or self.returns is None:
            return res
        return tuple(res)       # any sequence of ops comes back as a tuple (base.py:123-127)


def _result_ops(returns):
    if isinstance(returns, dict):
        return [returns[k] for k in returns]
    if isinstance(returns, ref.Op):
        return [returns]
    return list(returns) if returns is not None else []


class B200NgraphTransformer(Transformer):
    """The b200 back end behind the reference's transformer API."""

    transformer_name = "b200"
    default_rtol = 1e-05
    default_atol = 1e-08

    def __init__(self, **kwargs):
        # the reference base class expects no unknown keyword arguments
        shard_batch = kwargs.pop("shard_batch", True)
        # hetr-style graphs only: results that carry the parallel axis come back whole on every
        # replica (hetr gathers them to the host, ngraph/op_graph/comm_nodes.py: GatherRecvOp)
        gather_results = kwargs.pop("gather_results", True)
        if os.environ.get("B200NG_PLAN_ONLY") == "1":
            # plan and compile only (no device needed): lets the reference's own tests exercise
            # translation and planning on a machine without a GPU; calls then raise
            kwargs.setdefault("plan_only", True)
        self.impl = b2t.B200Transformer(**kwargs)
        self.translator = GraphTranslator(replicas=self.impl.comm.size, shard_batch=shard_batch,
                                          rank=self.impl.comm.rank)
        self.gather_results = bool(gather_results)
        self.computations = []
        self.finalized = False
        self._counts_as_flex = bool(self.impl.flex)
        if self._counts_as_flex:
            type(self)._flex_instances += 1

    # -- the API callers use ---------------------------------------------------------------------
    def computation(self, results, *parameters):
        return self.add_computation(ref.computation(results, *parameters))

    def add_computation(self, computation_op):
        if self.impl.finalized:
            raise ValueError("Cannot create computations from a finalized transformer")
        c = _PluginComputation(self, computation_op)
        self.computations.append(c)
        return c

    def initialize(self):
        self.impl.initialize()
        self.finalized = True

    def close(self):
        if self._counts_as_flex:
            self._counts_as_flex = False
            type(self)._flex_instances -= 1
        self.impl.close()

    _flex_instances = 0      # live transformers with flex16 storage (decides the class tolerance)

    @classmethod
    def get_default_tolerance(cls, desired):
        """(atol, rtol) the reference's test helpers widen their bars to
        (ngraph/testing/error_check.py:25-52 asks the CLASS): fp32 as its GPU transformer
        (gputransform.py:1043-1044), flex16 as its flex transformer (flexgputransform.py:80-103)."""
        if cls._flex_instances > 0:
            from . import flex as flexmod
            scale = flexmod.flex16.get_scale(float(np.max(np.abs(desired))))
            return scale * 8, 1e-2
        return cls.default_atol, cls.default_rtol

    # -- hooks of the abstract base that this back end does not route through -------------------
    @property
    def use_exop(self):
        return False

    def initialize_allocations(self):
        pass

    def get_tensor_view_value(self, op, host_tensor=None):
        """ngraph/transformers/base.py:546-558: the value a tensor of the graph holds now."""
        return self.impl.get_tensor_view_value(self.translator(op.tensor), host_tensor)

    def device_tensor(self, op):
        """The device tensor of a reference op (get / slicing / assignment from the host)."""
        return self.impl.device_tensor(self.translator(op.tensor))

    def host_to_device(self, computation, parameters, args):
        pass

    def device_to_host(self, computation, op, tensor=None):
        pass


class B200FlexNgraphTransformer(B200NgraphTransformer):
    """`make_transformer_factory('b200flex')`: flex16 storage with the reference flex
    transformer's own granularity -- every op's result is stored, and therefore quantised, as
    FlexGPUTransformer does with one kernel per op (flexgputransform.py:67-103) -- so that the
    reference's flex tests (tests/flex_tests, marker flex_only), whose expected values are exact
    mantissa-level facts of that granularity, run against it unchanged.  'b200' with flex=True is
    the same storage with fused kernels (intermediate values stay fp32)."""

    transformer_name = "b200flex"
    default_rtol = 1e-02

    def __init__(self, fixed_point=False, flex_verbose=False, collect_flex_data=False, **kwargs):
        kwargs.setdefault("flex", True)
        kwargs.setdefault("fuse", False)
        kwargs.update(fixed_point=fixed_point, flex_verbose=flex_verbose)
        super(B200FlexNgraphTransformer, self).__init__(**kwargs)

    @classmethod
    def get_default_tolerance(cls, desired):
        from . import flex as flexmod
        scale = flexmod.flex16.get_scale(float(np.max(np.abs(desired))))
        return scale * 8, 1e-2
