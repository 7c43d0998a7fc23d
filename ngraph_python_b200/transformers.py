"""The `b200` transformer: compiles an op graph into a list of CUDA launches and runs it.

Mirrors the reference's transformer API (ngraph/transformers/base.py): a registry of transformer
classes keyed by `transformer_name` (:265-279), `make_transformer`, `set_transformer_factory`,
`make_transformer_factory`, `transformer_choices` (:807-847), `Transformer.computation`
(:420-433) and `Computation.__call__` (:94-136).  What the reference's GPU backend does with
pycuda, NVRTC'd per-op kernels and maxas SASS (ngraph/transformers/gputransform.py:348-1148,
flexgputransform.py:67-371) is done here by hand-written sm_100a kernels behind the C ABI of
libb200ng.so; PyTorch only provides device memory, streams and pinned host buffers.

There is no CPU path: constructing the transformer without the shared library or without a CUDA
device raises.
"""
import collections
import math
import numbers

import numpy as np

from . import flex as flexmod
from . import fusion
from . import kernels
from . import lib
from . import comm as commmod
from . import tracing
from .op_graph import (AllReduceOp, AssignableTensorOp, AssignOp, Axes, AxesCastOp, BroadcastOp,
                       ConvolutionOp, DotOp, bprop_conv, update_conv,
                       BpropPoolOp, ElementWiseOp, LookupTableOp, Op, PoolingOp, ReductionOp, RngOp,
                       ReorderAxes, ReshapeOp, SequentialOp, TensorSliceOp, update_lut,
                       ViewOp, as_op, make_axes)


class UnsupportedTransformerException(Exception):
    """ngraph/transformers/base.py:37"""


# ---------------------------------------------------------------------------------------------
# storage
# ---------------------------------------------------------------------------------------------
class Buffer(object):
    """One device allocation; dense in `axes` order."""

    def __init__(self, name, axes, flex, persistent=False):
        self.name = name
        self.axes = make_axes(axes)
        self.size = self.axes.size
        self.flex = flex
        self.persistent = persistent
        self.tensor = None          # torch tensor, flat
        self.staging = None         # fp32 staging for flex host writes
        self.entry = None           # FlexEntry
        self.slot = -1              # flex table row of the data currently stored
        self.slot_write = -1        # row used by in-place writers (persistent tensors)
        self.init_array = None
        # flex16 tensors read by the implicit-GEMM convolution also exist as two byte planes
        self.plane_bytes = 0        # bytes of one plane (0: no planes wanted)
        self.planes = None          # torch uint8 allocation holding both planes
        self.planes_ptr = 0         # 1024-byte aligned start of the high plane
        self.planes_by_producer = False   # the kernel that writes the tensor writes the planes
        self.version = 0            # bumped whenever the contents change
        # planning state (per computation build)
        self.last_write_step = -1
        self.last_read_step = -1

    def ptr(self):
        return self.tensor.data_ptr()


class View(object):
    """A strided window on a buffer, described per named axis."""

    def __init__(self, buffer, axes, strides, offset=0):
        self.buffer = buffer
        self.axes = make_axes(axes)
        self.strides = tuple(int(s) for s in strides)
        self.offset = int(offset)

    @staticmethod
    def dense(buffer):
        strides, acc = [], 1
        for n in reversed(buffer.axes.lengths):
            strides.append(acc)
            acc *= n
        return View(buffer, buffer.axes, tuple(reversed(strides)))

    def stride_of(self, axis):
        for a, s in zip(self.axes, self.strides):
            if a == axis:
                return s
        return 0

    def key(self):
        return (id(self.buffer), tuple((a.name, s) for a, s in zip(self.axes, self.strides)
                                       if s != 0 and a.length != 1), self.offset)

    def is_dense(self):
        """The view walks the whole buffer in memory order (axes may have been renamed by a cast;
        the stride of an axis of length 1 is immaterial)."""
        if self.offset != 0:
            return False
        expect = 1
        for a, s in reversed(list(zip(self.axes, self.strides))):
            if a.length != 1 and s != expect:
                return False
            expect *= a.length
        return expect == self.buffer.size


# ---------------------------------------------------------------------------------------------
# steps (what the executor launches, in order)
# ---------------------------------------------------------------------------------------------
class EwStep(object):
    kind = "ew"

    def __init__(self, group):
        self.group = group
        self.index = group.index
        self.kernel = None
        self.in_views = []
        self.out_views = []      # elementwise outputs then reduction outputs
        self.out_targets = []    # (view, as byte planes?) per program result, in program order
        self.consts = []
        self.scratch = None

    def output_buffers(self):
        return [v.buffer for v in self.out_views]

    @property
    def launches(self):
        return self.kernel.launches


# ---------------------------------------------------------------------------------------------
class Computation(object):
    """A callable compiled from (returns, *parameters) (ngraph/transformers/base.py:44-136)."""

    def __init__(self, transformer, returns, parameters):
        self.transformer = transformer
        if isinstance(returns, (list, tuple)):
            self.returns_kind = type(returns)
            self.returns = [as_op(r) for r in returns]
        elif isinstance(returns, dict):
            raise ValueError("dict returns are not supported")
        elif returns is None:
            self.returns_kind = None
            self.returns = []
        else:
            self.returns_kind = Op
            self.returns = [as_op(returns)]
        self.parameters = [as_op(p) for p in parameters]
        for p in self.parameters:
            if not (isinstance(p, AssignableTensorOp) and p.is_input):
                raise ValueError("computation parameters must be placeholders or variables, "
                                 "got %r" % (p,))
        self.steps = None
        self.executor = None
        self.launches_per_call = 0
        self._comm_steps = []       # this computation's exchanges, in production order
        self._allreduce = None      # their arena and bucket plan (one per computation)

    # ---- compile -------------------------------------------------------------------------
    def _ordered_ops(self):
        order, seen = [], set()

        def visit(op):
            if op in seen:
                return
            seen.add(op)
            for a in op.all_deps:
                visit(a)
            order.append(op)
        for r in self.returns:
            visit(r)
        return order

    def build(self):
        t = self.transformer
        planner = _Planner(t, self)
        self.steps, self.return_views = planner.plan(self._ordered_ops(), self.returns)
        final = []
        for s in self.steps:
            final.extend(planner.finalize_step(s))     # (a step may bring copies that precede it)
        self.steps = final
        self._comm_steps = planner.comm_steps
        # (a parameter the results do not depend on still gets its tensor: callers pass a value)
        self.param_buffers = [t._view_of(p).buffer for p in self.parameters]
        t._allocate(self)
        for s in self.steps:
            if hasattr(s, "allocate"):
                s.allocate(t)
        self.launches_per_call = builtin_sum(s.launches for s in self.steps)
        self.written = planner.written_buffers
        self.executor = self._run_steps

    # ---- run -----------------------------------------------------------------------------
    def __call__(self, *args, **kwargs):
        t = self.transformer
        if self.steps is None:
            t.initialize()
        if t.plan_only:
            raise lib.B200Error("a plan_only transformer cannot run computations")
        feed = kwargs.pop("feed_dict", None)
        if feed is not None:
            args = [feed[p] for p in self.parameters]
        if len(args) != len(self.parameters):
            raise ValueError("Computation was expecting %d arguments, but was called with %d" %
                             (len(self.parameters), len(args)))
        views = [t._view_of(p) for p in self.parameters]
        for v, value in zip(views, args):
            t._stage(v, value)             # the input copies run while the host does the rest
        t._begin_call(self)
        for v in views:
            t._host_to_device(v, None, in_call=True, staged=True)
        traced = None
        if t.tracer is not None:
            traced = self._run_steps_traced()
        else:
            self.executor()
        # results, flex statistics and the status word come back with asynchronous copies and
        # ONE stream synchronisation
        pending = [t._device_to_host_async(v) for v in self.return_views]
        t._end_call(self)
        if traced is not None:
            t._collect_trace(self, traced)
        results = [t._finish_host(p) for p in pending]
        if self.returns_kind is Op:
            return results[0]
        if self.returns_kind is None:
            return None
        return tuple(results)

    def _run_steps(self):
        t = self.transformer
        for s in self.steps:
            t._launch_step(s)

    def _run_steps_traced(self):
        """The step list launched one by one, every step between two CUDA events."""
        t = self.transformer
        Event = t.torch.cuda.Event
        pairs = []
        for s in self.steps:
            e0, e1 = Event(enable_timing=True), Event(enable_timing=True)
            e0.record(t.stream)
            t._launch_step(s)
            e1.record(t.stream)
            pairs.append((s, e0, e1))
        return pairs

    def capture(self):
        """Records the step list into CUDA graphs and replays them from now on: one graph launch
        instead of one launch (plus tensor-map encoding) per kernel.  Call after the computation
        has run at least once, so that flex exponents exist and every kernel variant is compiled;
        flex scales live in a device table, so a replay picks up exponent changes.
        With several replicas and a communicator whose collectives can be recorded (the library's
        own NCCL group) the exchanges are nodes of the same graph: the communication stream forks
        from the recording stream where a bucket closes and joins it again before the bucket's
        first reader, so a training step is still ONE graph launch.  With any other communicator
        (torch.distributed) the exchanges stay outside: the step list is cut into segments at
        every point where a bucket is handed over or a reduced tensor is first needed, each
        segment is one graph, and the collectives are issued between the replays exactly where
        the step-by-step executor issues them."""
        t = self.transformer
        if self.steps is None or t.plan_only:
            raise lib.B200Error("run the computation once before capturing it")
        if t.flex and any(not b.entry.initialized for b in self.written):
            raise lib.B200Error("run the computation once before capturing it")
        torch = t.torch
        refreshable = [s for s in self.steps if hasattr(s, "refresh")]
        ar = self._allreduce
        has_comm = any(s.kind == "comm" for s in self.steps) and ar is not None and ar.comm.size > 1
        in_graph = has_comm and getattr(ar.comm, "capturable", False)
        if in_graph:
            has_comm = False             # one segment; the comm steps issue their collectives
        # -- segments ---------------------------------------------------------------------------
        segments, cur, made_here = [], None, set()

        def close():
            nonlocal cur, made_here
            if cur is not None and cur["steps"]:
                segments.append(cur)
            cur, made_here = None, set()
        for s in self.steps:
            needs = []
            if has_comm and s.kind != "comm":
                needs = [v.buffer.comm_key for v in s.in_views
                         if getattr(v.buffer, "comm_key", None) is not None]
            if any(k in made_here for k in needs):
                close()
            if cur is None:
                cur = {"steps": [], "wait": [], "comm": [], "graph": None}
            cur["steps"].append(s)
            for k in needs:
                if k not in cur["wait"]:
                    cur["wait"].append(k)
            if has_comm and s.kind == "comm":
                cur["comm"].append(s)
                made_here.add(s.key)
                if s.closes_bucket is not None:
                    close()
        close()
        # -- record ------------------------------------------------------------------------------
        torch.cuda.synchronize()
        before = t.kernel_launches
        t._allreduce = self._allreduce
        if t._allreduce is not None:
            t._allreduce.begin_call()
        t._recording = has_comm          # comm steps and waits: kernels only, no NCCL, no bookkeeping
        io_in_graph = False
        try:
            for seg in segments:
                if all(s.launches == 0 for s in seg["steps"]):
                    continue             # nothing to record (fp32 exchange markers)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    for s in seg["steps"]:
                        t._launch_step(s)
                    if in_graph:
                        ar.join_all()    # every forked stream is back before the recording ends
                    if seg is segments[-1]:
                        # the call's read-back rides in the graph: status word and flex
                        # statistics to pinned host memory, then the statistics cleared for the
                        # next call -- one graph launch and one synchronisation per call
                        t._publish()
                        io_in_graph = True
                seg["graph"] = g
        finally:
            t._recording = False
        per_call = t.kernel_launches - before
        self._graphs = [seg["graph"] for seg in segments]

        def replay():
            for s in refreshable:
                s.refresh(t)          # cached operand planes of tensors that changed since
            for seg in segments:
                for k in seg["wait"]:
                    ar.wait_for(k)
                if seg["graph"] is not None:
                    seg["graph"].replay()
                for cs in seg["comm"]:
                    ar.produced(cs.key)
                    if cs.closes_bucket is not None:
                        ar.bucket_ready(cs.closes_bucket)
            if in_graph:
                ar.graph_launched(t.stream)
            t.kernel_launches += per_call
            if io_in_graph:
                t._io_done = True
                t._stats_clean = t.flex
        self.executor = replay
        return self


builtin_sum = sum


# ---------------------------------------------------------------------------------------------
class _Planner(object):
    """Builds the step list of one computation: views, fusion groups, programs."""

    def __init__(self, transformer, computation):
        self.t = transformer
        self.comp = computation
        self.steps = []
        self.producer = {}        # op -> step index that produces its value
        self.group_of = {}        # EW/reduction op -> EwGroup
        self.consumers = collections.defaultdict(list)
        self.written_buffers = []
        self.conv_tails = {}       # ConvolutionOp -> dict(out, bias, residual, relu, ops)
        self.conv_tail_of = {}     # absorbed elementwise op -> its ConvolutionOp
        self.deferred = []         # re-quantisations of reduced tensors, placed at first use
        self.arg_override = {}     # op -> value args after register forwarding
        self.comm_steps = []       # exchanges of this computation, in the order they are placed
        self.last_assign = {}      # persistent tensor -> the AssignOp that last wrote all of it

    # -- helpers ------------------------------------------------------------------------------
    def _resolve(self, op):
        """Follows SequentialOp (and planner-made replacements) to the op that carries the value."""
        while True:
            if isinstance(op, SequentialOp):
                op = op.value_tensor
            elif op in self.t._alias:
                op = self.t._alias[op]
            else:
                return op

    def _is_scalar_const(self, op):
        return isinstance(op, AssignableTensorOp) and op.is_scalar_constant

    def _base_tensor(self, op):
        """(source op, view transform chain) for an argument: strips views."""
        op = self._resolve(op)
        chain = []
        while isinstance(op, ViewOp):
            chain.append(op)
            op = self._resolve(op.args[0])
        return op, chain

    def _new_step_index(self):
        return len(self.steps)

    def _value_args(self, op):
        """The arguments an elementwise op reads (an AssignOp: the assigned value), after the
        planner's register forwarding: a persistent tensor that the same kernel has just assigned
        is read from the register of that assignment instead of from memory."""
        if op in self.arg_override:
            return self.arg_override[op]
        return [op.args[1]] if isinstance(op, AssignOp) else list(op.args)

    def _forwarding(self, op, value_args):
        """(overridden args, group) when every in-place-written persistent tensor that `op` reads
        whole was last assigned by one and the same open kernel, else None."""
        new_args, group = list(value_args), None
        for i, a in enumerate(value_args):
            base, chain = self._base_tensor(a)
            if not isinstance(base, AssignableTensorOp) or base.is_scalar_constant:
                continue
            buf = self.t._buffer_of(base)
            if buf.last_write_step < 0:
                continue
            asg = self.last_assign.get(base)
            if chain or asg is None or self.group_of[asg].index != buf.last_write_step:
                return None
            if group is not None and self.group_of[asg] is not group:
                return None
            group = self.group_of[asg]
            new_args[i] = asg
        return (new_args, group) if group is not None else None

    # -- planning -----------------------------------------------------------------------------
    def _relu_masks_from_activations(self, ordered, returns):
        """`greater(x, 0)` -- the mask autodiff puts on the gradient of maximum(x, 0) -- reads the
        activation maximum(x, 0) instead of the pre-activation x where both exist: x > 0 exactly
        when max(x, 0) > 0, also for quantised values.  The pre-activation then has one reader
        left, so a convolution's ReLU (and the residual sum before it) folds into the
        convolution's epilogue in training as it does in inference, and x is never stored."""
        t = self.t
        if not (t.fuse and t.fuse_conv_tail):
            return ordered

        def is_zero(a):
            base, _ = self._base_tensor(a)
            return self._is_scalar_const(base) and float(np.asarray(base.initial_value)) == 0.0
        def key_of(a):
            base, _ = self._base_tensor(a)
            if isinstance(base, AssignableTensorOp):
                return None
            return t._view_of(self._resolve(a)).key()
        relu_of = {}
        for op in ordered:
            if isinstance(op, ElementWiseOp) and op.opname == "maximum" and len(op.args) == 2:
                for i in (0, 1):
                    if is_zero(op.args[1 - i]) and key_of(op.args[i]) is not None:
                        relu_of.setdefault((key_of(op.args[i]), op.args[i].axes), op)
        if not relu_of:
            return ordered
        out = []
        for op in ordered:
            new = None
            if isinstance(op, ElementWiseOp) and op.opname == "gt" and len(op.args) == 2 and \
                    is_zero(op.args[1]):
                act = relu_of.get((key_of(op.args[0]), op.args[0].axes))
                if act is not None and act.axes == op.args[0].axes:
                    new = ElementWiseOp("gt", (act, op.args[1]))
            if new is None:
                out.append(op)
            else:
                t._alias[op] = new
                out.append(new)
        return out

    def _sink_to_consumer(self, ordered, returns):
        """Moves an elementwise op whose value has a single reader, itself elementwise over the
        same axes, to just before that reader, so that the two share a kernel and the value is
        never stored (the masks `x > 0` of back-propagation are the typical case: computed where
        the reference's ordering puts them they would be written out and read back).  Only ops
        over tensors that nothing overwrites are moved."""
        if not self.t.fuse:
            return ordered
        returned = set(self._base_tensor(r)[0] for r in returns)
        # (a SequentialOp that merely lists an op orders it, it does not read it: the op may
        # run later as long as what it reads cannot change, which is checked below)
        readers = collections.defaultdict(list)
        for op in ordered:
            if isinstance(op, SequentialOp):
                continue
            for a in op.args:
                readers[self._base_tensor(a)[0]].append(op)
        held = collections.defaultdict(list)      # reader -> ops to emit right before it
        for op in ordered:
            if not isinstance(op, ElementWiseOp) or op in returned or op.opname == "assign":
                continue
            rs = readers.get(op, ())
            if len(rs) != 1 or not isinstance(rs[0], ElementWiseOp) or rs[0].axes != op.axes:
                continue
            movable = True
            for a in op.args:
                base, _ = self._base_tensor(a)
                if isinstance(base, AssignableTensorOp) and not base.is_scalar_constant and \
                        not base.is_constant:
                    movable = False
            if movable:
                held[rs[0]].append(op)
        if not held:
            return ordered
        moved = set(o for ops in held.values() for o in ops)
        out = []

        def emit(op):
            for o in held.get(op, ()):
                emit(o)
            out.append(op)
        for op in ordered:
            if op not in moved:
                emit(op)
        return out

    def plan(self, ordered, returns):
        ordered = self._relu_masks_from_activations(ordered, returns)
        ordered = self._sink_to_consumer(ordered, returns)
        for op in ordered:
            for a in op.args:
                self.consumers[self._base_tensor(a)[0]].append(op)
        returned = set(self._base_tensor(r)[0] for r in returns)
        self.returned = returned
        for buf in self.t._buffers.values():
            buf.last_write_step = -1
            buf.last_read_step = -1
        self._find_conv_tails(ordered)
        for op in ordered:
            if op in self.conv_tail_of:
                # part of a convolution layer's elementwise tail: the layer is placed, as one step,
                # where its last op stands (every operand of the tail exists by then)
                conv = self.conv_tail_of[op]
                if self.conv_tails[conv]["out"] is op:
                    self._place_other(conv)
                continue
            if isinstance(op, ConvolutionOp) and op in self.conv_tails:
                continue
            if isinstance(op, (ElementWiseOp, ReductionOp, AssignOp)):
                self._place_ew(op)
            elif isinstance(op, AllReduceOp):
                self._place_allreduce(op)
            elif isinstance(op, (AssignableTensorOp, ViewOp, SequentialOp)):
                continue
            else:
                self._place_other(op)
        while self.deferred:                       # reduced tensors that are only returned
            self._place_ew(self.deferred.pop(0))
        # replacements made while placing (allreduce) change what the returns resolve to
        self.returned = set(self._base_tensor(r)[0] for r in returns)
        # decide what each group materialises
        for step in self.steps:
            if step.kind == "ew":
                self._collect_outputs(step)
        steps = [s for s in self.steps if s.kind != "ew" or s.out_ops]
        return_views = [self.t._view_of(self._resolve(r)) for r in returns]
        return steps, return_views

    def _place_ew(self, op):
        is_assign = isinstance(op, AssignOp)
        is_red = isinstance(op, ReductionOp)
        self._place_deferred_for(op.args[1:] if is_assign else op.args)
        if is_assign:
            target = op.args[0]
            value_args = [op.args[1]]
            iter_axes = target.axes
            tbuf = self.t._view_of(target).buffer
        else:
            value_args = list(op.args)
            iter_axes = op.args[0].axes if is_red else op.axes
        # (a flex16 reader must see the stored, quantised value -- the Kahan term of the optimizer
        # exists to capture exactly that quantisation error: there the register is re-quantised
        # with the exponent of the store, see _finalize_ew)
        fwd = self._forwarding(op, value_args) if (self.t.fuse and self.t.forward_inplace) else None
        if fwd is not None:
            # try the kernel that made the in-place writes this op reads: its registers still
            # hold the values, so the op can run there instead of in a later launch
            self.arg_override[op] = fwd[0]
            if self._place_ew_with(op, is_assign, is_red, iter_axes, fwd[0], only=fwd[1]):
                return
            del self.arg_override[op]
        self._place_ew_with(op, is_assign, is_red, iter_axes, value_args, only=None)

    def _place_ew_with(self, op, is_assign, is_red, iter_axes, value_args, only):
        if is_assign:
            target = op.args[0]
            tbuf = self.t._view_of(target).buffer
        lower = -1
        for a in value_args:
            base, chain = self._base_tensor(a)
            if isinstance(base, AssignableTensorOp):
                if not base.is_scalar_constant:
                    lws = self.t._buffer_of(base).last_write_step
                    if lws >= 0:
                        lower = max(lower, lws + 1)    # must see the in-place write
            elif base in self.producer:
                direct = not chain and not isinstance(base, ReductionOp) and base in self.group_of
                lower = max(lower, self.producer[base] + (0 if direct else 1))
        if is_assign:
            lower = max(lower, tbuf.last_write_step, tbuf.last_read_step)
        # candidate groups: the latest open groups that run late enough for every dependency;
        # independent chains over the same iteration space end up in one kernel this way
        group = None
        tried = 0
        for step in reversed(self.steps if self.t.fuse else []):
            if step.index < lower or tried >= 6:
                break
            if step.kind != "ew":
                continue
            tried += 1
            cand = step.group
            if only is not None and cand is not only:
                continue
            if not self._can_join(cand, op, iter_axes, is_red):
                continue
            if is_assign and tbuf.last_read_step == cand.index:
                # the group already reads the target: in-place is safe only element for element
                tv = self.t._view_of(target)
                if any(v.buffer is tbuf and v.key() != tv.key() for v in cand.ext_inputs):
                    continue
            group = cand
            break
        if group is None and only is not None:
            return False
        if group is None:
            group = fusion.EwGroup(self._new_step_index(), iter_axes)
            step = EwStep(group)
            step.out_ops = []
            self.steps.append(step)
        group.add(op)
        if is_red or is_assign or op in self.returned:
            group.stored.add(op)
        if is_red:
            group.red_axes = op.reduction_axes
        self.group_of[op] = group
        self.producer[op] = group.index
        # external loads of this op
        for a in value_args:
            base, chain = self._base_tensor(a)
            if self._is_scalar_const(base):
                group.n_consts += 1
                continue
            if group.has(base) and not chain and not isinstance(base, ReductionOp):
                continue
            if base in self.group_of:
                self.group_of[base].stored.add(base)     # consumed outside its own kernel
            v = self.t._view_of(self._resolve(a))
            if not any(v.key() == w.key() for w in group.ext_inputs):
                group.ext_inputs.append(v)
                # a persistent tensor read after an in-place write of this computation carries
                # the exponent chosen for that write
                group.after_write[v.key()] = isinstance(base, AssignableTensorOp) and \
                    self.t._buffer_of(base).last_write_step >= 0
            if isinstance(base, AssignableTensorOp):
                b = self.t._buffer_of(base)
                b.last_read_step = max(b.last_read_step, group.index)
        if is_assign:
            tbuf.last_write_step = group.index
            whole = self.t._view_of(target).is_dense()
            self.last_assign[self._base_tensor(target)[0]] = op if whole else None
        return True

    def _can_join(self, g, op, iter_axes, is_red):
        if g.iter_axes != iter_axes:
            return False
        if is_red:
            if g.red_axes is not None and g.red_axes != op.reduction_axes:
                return False
        new_inputs = 0
        for a in self._value_args(op):
            base, chain = self._base_tensor(a)
            if g.has(base) and isinstance(base, ReductionOp):
                return False     # needs a value that exists only after the whole reduction
            if self._is_scalar_const(base) or (g.has(base) and not chain):
                continue
            new_inputs += 1
        if len(g.ext_inputs) + new_inputs > fusion.MAX_IN:
            return False
        # the iteration space must still fold onto the kernel's three axes
        views = list(g.ext_inputs)
        for a in self._value_args(op):
            base, chain = self._base_tensor(a)
            if self._is_scalar_const(base) or (g.has(base) and not chain):
                continue
            views.append(self.t._view_of(self._resolve(a)))
        red_axes = op.reduction_axes if is_red else (g.red_axes or Axes())
        strides = [[v.stride_of(a) for a in iter_axes] for v in views]
        dense, acc = [], 1
        for n in reversed(iter_axes.lengths):
            dense.append(acc)
            acc *= n
        strides.append(list(reversed(dense)))
        try:
            cl, cs, cr = fusion.collapse_dims(list(iter_axes.lengths), strides,
                                              [a in red_axes for a in iter_axes])
            fusion.map_to_abc(cl, cs, cr)
        except ValueError:
            return False
        if len(g.members) + 1 > fusion.MAX_OPS or g.n_consts + 2 > fusion.MAX_CONST:
            return False
        if len(g.stored) + 1 > fusion.MAX_OUT - 1:      # one spare for a later outside consumer
            return False
        if self._prospective_outputs(g, op) > fusion.MAX_OUT:
            return False
        return True

    def _prospective_outputs(self, g, op):
        """How many values the kernel would have to store if `op` joined it now: assignments,
        reductions, returned values, and values read outside the kernel (a reader that has not
        been placed yet counts as outside, which errs on the safe side)."""
        members = list(g.members) + [op]
        inside = set(members)
        count = 0
        for m in members:
            if isinstance(m, (AssignOp, ReductionOp)) or m in self.returned:
                count += 1
                continue
            for c in self.consumers.get(m, ()):
                direct = any(self._base_tensor(a)[0] is m and not self._base_tensor(a)[1]
                             for a in c.args)
                if c not in inside or not direct:
                    count += 1
                    break
        return count

    def _place_allreduce(self, op):
        """fp32: the producer's buffer is placed in the communication arena and reduced in
        place.  flex16: the int16 gradient is de-quantised into an fp32 arena slot, reduced
        there, and re-quantised by an ordinary fused kernel, so every replica derives the same
        exponent from the same reduced values."""
        t = self.t
        src, chain = self._base_tensor(op.args[0])
        if chain or isinstance(src, AssignableTensorOp):
            raise ValueError("Unhandled op: allreduce of a view or of a variable: {}".format(op))
        if src in self.group_of:
            self.group_of[src].stored.add(src)
        index = self._new_step_index()
        src_view = t._view_of(src)
        if not t.flex:
            buf = src_view.buffer
            buf.in_arena = True
            buf.comm_key = id(buf)
            step = kernels.CommStep(index, op, t, None, buf)
            t._alias[op] = src                 # consumers read the same (now reduced) buffer
            t._views[op] = src_view
            self.producer[src] = max(self.producer.get(src, -1), index)
        else:
            from .op_graph import AssignableTensorOp as _A
            staging = _A(op.axes, name=op.name + "_f32")
            sbuf = Buffer(staging.name, op.axes, False, persistent=True)
            sbuf.in_arena = True
            sbuf.comm_key = id(sbuf)
            sbuf.entry = None
            t._buffers[staging] = sbuf
            step = kernels.CommStep(index, op, t, src_view, sbuf)
            sbuf.last_write_step = index
            requant = ElementWiseOp("assign", (staging,))
            t._alias[op] = requant
            # whoever consumes the allreduce consumes the re-quantised tensor: without this a
            # consumer in a later kernel would find nothing stored
            self.consumers[requant] = list(self.consumers.get(op, ()))
        step.reduce_func = op.reduce_func
        self.steps.append(step)
        self.producer[op] = index
        self.comm_steps.append(step)
        if t.flex:
            # placed when its first consumer is: a re-quantisation right here would need the
            # reduced values at once and force one small exchange per tensor instead of one per
            # bucket overlapped with the rest of back-propagation
            self.deferred.append(requant)

    def _find_conv_tails(self, ordered):
        """flex16, implicit-GEMM convolutions: folds `+ bias[channel]`, `+ residual` and
        `maximum(., 0)` that follow a convolution -- each the only reader of the value before it
        -- into the convolution step (evaluated in the tile kernel's epilogue; the reference's
        kernels carry bias / relu flags for the same purpose, ngraph/transformers/gpu/conv.py)."""
        t = self.t
        if not (t.flex and t.fuse and t.fuse_conv_tail):
            return
        for conv in ordered:
            if not isinstance(conv, ConvolutionOp):
                continue
            try:
                ok = lib.conv_planes_info(kernels._conv_dims_of(conv, t), lib.CONV_FPROP)[0]
            except Exception:
                ok = False
            if not ok:
                continue
            info = dict(out=None, bias=None, residual=None, relu=False, ops=[])
            cur = conv
            chan = conv.axes[0].length
            while True:
                # (a SequentialOp only orders: it reads nothing)
                readers = [r for r in self.consumers.get(cur, ())
                           if not isinstance(r, (ViewOp, SequentialOp))]
                if len(readers) != 1 or cur in self.returned:
                    break
                nxt = readers[0]
                if not isinstance(nxt, ElementWiseOp) or len(nxt.args) != 2:
                    break
                if nxt in self.conv_tail_of:
                    break        # the sum of two branches belongs to one of them only
                mine = [i for i, a in enumerate(nxt.args) if self._base_tensor(a)[0] is cur]
                if len(mine) != 1:
                    break
                other = nxt.args[1 - mine[0]]
                obase, ochain = self._base_tensor(other)
                # (same shape up to axes of length 1: the reference's layers drop the unit depth
                # axis of the result with a slice before the activation)
                if [n for n in nxt.axes.lengths if n != 1] != [n for n in conv.axes.lengths if n != 1]:
                    break
                if nxt.opname == "add" and not info["relu"]:
                    is_bias = (len(obase.axes) == 1 and obase.axes[0].length == chan and
                               obase.axes[0] == nxt.axes[0] and not self._is_scalar_const(obase))
                    if ochain:
                        # a view of the other tensor that still walks it in memory order (the
                        # reference's layers drop a unit axis with a slice)
                        oview = t._view_of(self._resolve(other))
                        same = oview.is_dense() and oview.axes == nxt.axes
                    else:
                        same = (tuple(obase.axes.lengths) == tuple(nxt.axes.lengths)
                                and obase.axes == nxt.axes)
                    if is_bias and info["bias"] is None and info["residual"] is None:
                        info["bias"] = obase
                    elif same and info["residual"] is None and not isinstance(obase, AssignableTensorOp):
                        info["residual"] = other if ochain else obase
                    else:
                        break
                elif nxt.opname == "maximum" and not info["relu"] and self._is_scalar_const(obase) \
                        and float(np.asarray(obase.initial_value)) == 0.0:
                    info["relu"] = True
                else:
                    break
                info["ops"].append(nxt)
                cur = nxt
            if info["ops"]:
                info["out"] = cur
                self.conv_tails[conv] = info
                for o in info["ops"]:
                    self.conv_tail_of[o] = conv

    def _place_deferred_for(self, args):
        for a in args:
            base, _ = self._base_tensor(a)
            if base in self.deferred:
                self.deferred.remove(base)
                self._place_ew(base)

    def _place_other(self, op):
        """Dense contractions and pooling: one step each, never fused with neighbours."""
        tail = self.conv_tails.get(op) if isinstance(op, ConvolutionOp) else None
        reads = list(op.args)
        if tail:
            reads += [x for x in (tail["bias"], tail["residual"]) if x is not None]
        self._place_deferred_for(reads)
        # Operands these kernels cannot take as they lie (a sliced or reordered view where a dense
        # tensor is needed; a dot operand that does not fold to two dimensions) are first copied
        # into dense temporaries by the strided copy kernel -- what the reference's layout pass
        # does with DimshuffleOps (ngraph/transformers/passes/layout.py:282-339).  The copies
        # stand in for the operands' views only while this step is built.
        saved = {}
        try:
            if isinstance(op, DotOp):
                try:
                    kernels.GemmStep(self._new_step_index(), op, self.t)
                except ValueError:
                    x, y = op.args
                    red = [a for a in x.axes if a in op.reduction_axes]
                    self._densify(x, list(op.x_out_axes) + red, saved)
                    self._densify(y, red + list(op.y_out_axes), saved)
            elif isinstance(op, (ConvolutionOp, bprop_conv, update_conv, PoolingOp, BpropPoolOp,
                                 LookupTableOp, update_lut)):
                for a in op.args:
                    if not self.t._view_of(a).is_dense():
                        self._densify(a, list(self.t._view_of(a).axes), saved)
            step = self._make_other_step(op, tail)
        finally:
            for key, old in saved.items():
                if old is None:
                    self.t._views.pop(key, None)
                else:
                    self.t._views[key] = old
        index = step.index
        self._register_other(op, step, reads, tail)

    def _densify(self, arg, axes, saved):
        """Appends a copy step that lays `arg` out dense over `axes` and makes the copy stand in
        for the argument's view until the caller restores `saved`."""
        t = self.t
        key = arg
        while isinstance(key, SequentialOp) or key in t._alias:
            key = key.value_tensor if isinstance(key, SequentialOp) else t._alias[key]
        view = t._view_of(key)
        pre, nv = self._dense_copy_of(view, make_axes(axes), self._new_step_index(), expand=True)
        base, _ = self._base_tensor(arg)
        if base in self.group_of:
            self.group_of[base].stored.add(base)
        if isinstance(base, AssignableTensorOp) and not base.is_scalar_constant:
            b = t._buffer_of(base)
            b.last_read_step = max(b.last_read_step, pre.index)
            if t.flex and b.last_write_step >= 0:
                nv.buffer.slot = b.slot_write      # the copy carries what the in-place write stored
        self.steps.append(pre)
        if key not in saved:
            saved[key] = t._views.get(key)
        t._views[key] = nv

    def _make_other_step(self, op, tail):
        index = self._new_step_index()
        if isinstance(op, DotOp):
            step = kernels.GemmStep(index, op, self.t)
        elif isinstance(op, ConvolutionOp):
            step = kernels.ConvStep(index, op, self.t, epilogue=tail)
            if tail:
                step.out_op = tail["out"]
                self.producer[tail["out"]] = index
                for o in tail["ops"]:
                    self.producer[o] = index
        elif isinstance(op, bprop_conv):
            step = kernels.ConvBpropStep(index, op, self.t)
        elif isinstance(op, update_conv):
            step = kernels.ConvUpdateStep(index, op, self.t)
        elif isinstance(op, PoolingOp):
            step = kernels.PoolStep(index, op, self.t)
        elif isinstance(op, BpropPoolOp):
            step = kernels.PoolBpropStep(index, op, self.t)
        elif isinstance(op, LookupTableOp):
            step = kernels.LutStep(index, op, self.t)
        elif isinstance(op, update_lut):
            step = kernels.LutUpdateStep(index, op, self.t)
        elif isinstance(op, RngOp):
            step = kernels.RngStep(index, op, self.t)
        else:
            raise ValueError("Unhandled op: {}".format(op))
        return step

    def _register_other(self, op, step, reads, tail):
        index = step.index
        if isinstance(op, RngOp):
            reads = []                 # the argument only supplies the axes
        # the step must come after everything its arguments depend on; steps are appended in
        # dependency order, so only in-place writes of persistent tensors need recording
        for a in reads:
            base, _ = self._base_tensor(a)
            if base in self.group_of:
                self.group_of[base].stored.add(base)
            if isinstance(base, AssignableTensorOp) and not base.is_scalar_constant:
                b = self.t._buffer_of(base)
                b.last_read_step = max(b.last_read_step, index)
                step.reads_after_write = getattr(step, "reads_after_write", set())
                if b.last_write_step >= 0:
                    step.reads_after_write.add(id(b))
        self.steps.append(step)
        self.producer[op] = index
        self.t._need_scratch(step.scratch_bytes)
        for b in step.output_buffers():
            if b not in self.written_buffers:
                self.written_buffers.append(b)

    def _only_plane_readers(self, m):
        """True when every reader of the value m is a convolution that takes it as byte planes
        (then the int16 copy need not be written at all)."""
        if m in self.returned:
            return False
        readers = [r for r in self.consumers.get(m, ()) if not isinstance(r, ViewOp)]
        if not readers:
            return False
        buf = self.t._view_of(m).buffer
        steps = getattr(buf, "plane_steps", ())
        for c in readers:
            st = [x for x in steps if x.op is c]
            if not st:
                return False
            for i, a in enumerate(c.args):
                if self._base_tensor(a)[0] is m and i != st[0].plane_arg:
                    return False
        return True

    def _collect_outputs(self, step):
        """Which values of the group must be stored: those used by another step or returned."""
        g = step.group
        outs = []
        for m in g.members:
            if isinstance(m, AssignOp):
                outs.append(m)
                continue
            needed = m in self.returned or isinstance(m, ReductionOp)
            if not needed:
                for c in self.consumers.get(m, ()):
                    cg = self.group_of.get(c)
                    direct = any(self._base_tensor(a)[0] is m and not self._base_tensor(a)[1]
                                 for a in c.args)
                    if cg is not g or not direct:
                        needed = True
                        break
            if needed:
                outs.append(m)
        if len(outs) > fusion.MAX_OUT:
            raise ValueError("Unhandled op: fused kernel with %d outputs" % len(outs))
        step.out_ops = outs
        for m in outs:
            if not isinstance(m, AssignOp):
                self.t._view_of(m)       # creates the buffer

    # -- program construction -------------------------------------------------------------------
    def finalize_step(self, step):
        """Builds the step's program; returns the steps that take its place in the list."""
        if step.kind == "ew":
            return self._finalize_ew(step)
        if getattr(step, "epi", None):
            # a fused convolution writes the byte planes of its result itself when the next
            # convolution wants them, and the int16 tensor only if someone reads that
            buf = step.out_views[0].buffer
            if buf.plane_bytes > 0:
                buf.planes_by_producer = True
                step.write_int16 = not self._only_plane_readers(step.out_op)
        return [step]

    def _pure_copy(self, step):
        """(source view, destination view) when the kernel would do nothing but copy one tensor
        into another -- value_of / a materialised reorder, or an fp32 AssignOp -- else None."""
        g = step.group
        if len(g.members) != 1 or len(step.out_ops) != 1 or len(g.ext_inputs) != 1:
            return None
        m = g.members[0]
        if isinstance(m, AssignOp):
            if self.t.flex:
                return None      # the target has an exponent of its own: values are re-quantised
            dst = self.t._view_of(m.args[0])
        elif isinstance(m, ElementWiseOp) and m.opname == "assign":
            dst = self.t._view_of(m)
        else:
            return None
        args = self._value_args(m)
        base, _ = self._base_tensor(args[0])
        if self._is_scalar_const(base):
            return None
        src = g.ext_inputs[0]
        if src.buffer.flex != dst.buffer.flex:
            return None
        if any(src.stride_of(a) == 0 and a.length != 1 for a in g.iter_axes):
            return None          # a broadcasting fill: the elementwise kernel does that well
        return src, dst

    def _dense_copy_of(self, view, iter_axes, index, expand=False):
        """A dimshuffle step that lays `view` out dense in iteration order, and the new view.
        expand: axes the view only broadcasts along are written out too."""
        t = self.t
        axes = [a for a in iter_axes if expand or view.stride_of(a) != 0 or a.length == 1]
        tmp = Buffer("dimshuffle_%d" % len(t._buffers), axes, view.buffer.flex)
        if view.buffer.flex:
            t._share_entry(tmp, view.buffer)
        t._buffers[object()] = tmp
        new_view = View.dense(tmp)
        return kernels.DimshuffleStep(index, None, t, view, new_view, make_axes(axes)), new_view

    def _finalize_ew(self, step):
        t = self.t
        g = step.group
        iter_axes = g.iter_axes
        red_axes = g.red_axes if g.red_axes is not None else Axes()
        lengths = list(iter_axes.lengths)
        reduced = [a in red_axes for a in iter_axes]
        ew_outs = [m for m in step.out_ops if not isinstance(m, ReductionOp)]
        red_outs = [m for m in step.out_ops if isinstance(m, ReductionOp)]
        out_views = []
        for m in ew_outs + red_outs:
            out_views.append(t._view_of(m.args[0]) if isinstance(m, AssignOp) else t._view_of(m))
        pre_steps = []
        key_views = list(g.ext_inputs)      # what the ops' arguments resolve to (looked up by key)

        def fold():
            sl = [[v.stride_of(a) for a in iter_axes] for v in list(g.ext_inputs) + out_views]
            red = [a in red_axes for a in iter_axes]
            clen, cstr, cred = fusion.collapse_dims(list(iter_axes.lengths), sl, red)
            return (clen, cstr) + fusion.map_to_abc(clen, cstr, cred)
        copy = self._pure_copy(step)
        folded = None
        try:
            folded = fold()
        except ValueError:
            if copy is None:
                # More non-mergeable axes than the kernel has, or reduced axes that do not lie
                # together: walk the kept axes first and the reduced ones last, and lay the
                # inputs that are to blame out dense in that order first (the reference's layout
                # pass inserts DimshuffleOps for the same purpose,
                # ngraph/transformers/passes/layout.py:282-339)
                if any(reduced):
                    iter_axes = make_axes([a for a in iter_axes if a not in red_axes] +
                                          [a for a in iter_axes if a in red_axes])
                for i, v in enumerate(list(g.ext_inputs)):
                    own = [a for a in iter_axes if v.stride_of(a) != 0 or a.length == 1]
                    expect, dense = 1, True
                    for a in reversed(own):
                        dense = dense and (a.length == 1 or v.stride_of(a) == expect)
                        expect *= a.length
                    if dense:
                        continue
                    pre, nv = self._dense_copy_of(v, iter_axes, step.index)
                    g.after_write[nv.key()] = g.after_write.get(v.key(), False)
                    g.ext_inputs[i] = nv
                    pre_steps.append(pre)
                folded = fold()                 # raises as before if that was not the obstacle
        if copy is not None:
            src, dst = copy
            # a transposing copy (source not contiguous along the destination's fastest axis), or
            # one over more axes than the elementwise kernel folds: the tiled copy kernel
            transposing = folded is None or (len(folded[0]) >= 1 and folded[1][0][-1] != 1)
            if folded is None or (transposing and src.buffer.size >= 1024):
                m = g.members[0]
                if t.flex:
                    t._share_entry(dst.buffer, src.buffer)
                return [kernels.DimshuffleStep(step.index, m, t, src, dst, iter_axes)]
        clen, cstr, dims, abc, mode = folded
        in_views = list(g.ext_inputs)
        # registers
        reg = {}
        consts = []
        const_reg = {}
        ops = []
        n_in = len(in_views)

        def input_index(view):
            for i, w in enumerate(key_views):
                if w.key() == view.key():
                    return i
            raise KeyError(view)

        pending = []     # (dst op, opname, [arg descriptors])
        for m in g.members:
            if isinstance(m, ReductionOp):
                # a reduction of a broadcast scalar constant reads the constant's register
                base, _ = self._base_tensor(self._value_args(m)[0])
                if self._is_scalar_const(base):
                    val = float(np.asarray(base.initial_value))
                    if val not in const_reg:
                        const_reg[val] = len(consts)
                        consts.append(val)
                continue
            args = self._value_args(m)
            descs = []
            for a in args:
                base, chain = self._base_tensor(a)
                if self._is_scalar_const(base):
                    val = float(np.asarray(base.initial_value))
                    if val not in const_reg:
                        const_reg[val] = len(consts)
                        consts.append(val)
                    descs.append(("c", const_reg[val]))
                elif g.has(base) and not chain and not isinstance(base, ReductionOp):
                    descs.append(("r", base))
                else:
                    descs.append(("i", input_index(t._view_of(self._resolve(a)))))
            pending.append((m, "assign" if isinstance(m, AssignOp) else m.opname, descs))
        n_const = len(consts)

        def resolve(d):
            if d[0] == "c":
                return n_in + d[1]
            if d[0] == "i":
                return d[1]
            return reg[d[1]]
        # flex16: an assignment whose value a later op of this kernel reads from the register is
        # followed by a requant op, so that the reader sees what the tensor now holds
        read_back = set(d[1] for _, _, descs in pending for d in descs
                        if d[0] == "r" and isinstance(d[1], AssignOp))
        requants = []    # (position in ops, AssignOp): the result index is known further down
        for m, name, descs in pending:
            a = resolve(descs[0])
            b = resolve(descs[1]) if len(descs) > 1 else None
            ops.append((name, a, b))
            reg[m] = n_in + n_const + len(ops) - 1
            if t.flex and m in read_back and t._view_of(m.args[0]).buffer.flex:
                ops.append(("requant", reg[m], None))
                requants.append((len(ops) - 1, m))
                reg[m] = n_in + n_const + len(ops) - 1

        if t.flex:
            ops = _fuse_sigmoid(ops, n_in, consts)

        def tdesc(view, st):
            fx = view.buffer.flex
            return dict(dtype=lib.FLEX16 if fx else lib.F32, strides=st)
        inputs = []
        for v, st in zip(in_views, abc[:n_in]):
            d = tdesc(v, st)
            d["slot"] = -1
            if v.buffer.flex:
                d["slot"] = v.buffer.slot_write if g.after_write.get(v.key()) else v.buffer.slot
            inputs.append(d)
        outs, reds = [], []
        out_targets, red_targets = [], []
        result_index = {}
        for k, (m, v) in enumerate(zip(ew_outs + red_outs, out_views)):
            d = tdesc(v, abc[n_in + k])
            d["slot"] = t._write_slot(v.buffer) if v.buffer.flex else -1
            if isinstance(m, ReductionOp):
                src = self._value_args(m)[0]
                base, chain = self._base_tensor(src)
                if g.has(base) and not chain:
                    d["reg"] = reg[base]
                elif self._is_scalar_const(base):
                    d["reg"] = n_in + const_reg[float(np.asarray(base.initial_value))]
                else:
                    d["reg"] = input_index(t._view_of(self._resolve(src)))
                if mode == lib.REDUCE_NONE:
                    # every reduced axis has length 1: the reduction is a copy
                    if m.redop in ("argmax", "argmin"):
                        raise ValueError("Unhandled op: {} over axes of length 1".format(m.redop))
                    ops.append(("assign", d["reg"], None))
                    d["reg"] = n_in + n_const + len(ops) - 1
                    outs.append(d)
                    out_targets.append((v, False))
                    continue
                d["redop"] = m.redop
                reds.append(d)
                red_targets.append((v, False))
            else:
                d["reg"] = reg[m]
                buf = v.buffer
                wants = (buf.flex and buf.plane_bytes > 0 and not isinstance(m, AssignOp) and
                         v.is_dense() and len(outs) + len(red_outs) + 2 <= fusion.MAX_OUT)
                if wants:
                    # the convolutions that read this tensor take it as two byte planes: write
                    # them here instead of running a split pass in front of every convolution
                    pd = dict(d)
                    pd["dtype"] = lib.FLEX16_PLANES
                    pd["plane_bytes"] = buf.plane_bytes
                    outs.append(pd)
                    out_targets.append((v, True))
                    buf.planes_by_producer = True
                if not (wants and self._only_plane_readers(m)):
                    result_index[m] = len(outs)
                    outs.append(d)
                    out_targets.append((v, False))
        for at, m in requants:
            ops[at] = ("requant", ops[at][1], result_index[m])
        # which results' stored form each result depends on (through requant ops): a tensor that
        # is written for the first time gets its exponent only after those it depends on
        dep = {}
        for i, (name, a, b) in enumerate(ops):
            r = n_in + n_const + i
            if name == "requant":
                dep[r] = dep.get(a, 0) | (1 << b)
            else:
                dep[r] = dep.get(a, 0) | (dep.get(b, 0) if b is not None and name != "onehot" else 0)
        step.requant_deps = [dep.get(d["reg"], 0) & ~(1 << k if k < len(outs) else 0)
                             for k, d in enumerate(outs + reds)]
        prog = lib.make_program(dims, inputs, consts, ops, outs, reds, mode)
        step.kernel = lib.PlannedKernel(prog, self.t.flex) if self.t.plan_only else lib.EwKernel(prog)
        step.in_views = in_views
        step.out_views = out_views
        step.out_targets = out_targets + red_targets
        step.consts = consts
        step.scratch_bytes = step.kernel.scratch_bytes
        t._need_scratch(step.scratch_bytes)
        for v in out_views:
            if v.buffer not in self.written_buffers:
                self.written_buffers.append(v.buffer)
        return pre_steps + [step]


def _reshape_strides(old_shape, old_strides, new_shape):
    """Element strides under which `new_shape` walks the same elements in the same order as
    (old_shape, old_strides), or None when that needs a copy.  Axes of extent 1 are free; a
    group of old axes can be re-cut only where it is contiguous within itself."""
    olds = [(n, st) for n, st in zip(old_shape, old_strides) if n != 1]
    out = []
    oi = 0
    ni = 0
    news = list(new_shape)
    while ni < len(news):
        if news[ni] == 1:
            out.append(0)
            ni += 1
            continue
        if oi >= len(olds):
            return None
        # grow a group of old axes and a group of new axes until their sizes agree
        o_size, n_size = olds[oi][0], news[ni]
        o_end, n_end = oi + 1, ni + 1
        while o_size != n_size:
            if o_size < n_size:
                if o_end >= len(olds):
                    return None
                o_size *= olds[o_end][0]
                o_end += 1
            else:
                while n_end < len(news) and news[n_end] == 1:
                    n_end += 1
                if n_end >= len(news):
                    return None
                n_size *= news[n_end]
                n_end += 1
        # the old group must be contiguous within itself
        for k in range(oi, o_end - 1):
            if olds[k][1] != olds[k + 1][1] * olds[k + 1][0]:
                return None
        st = olds[o_end - 1][1]
        part = []
        for k in range(n_end - 1, ni - 1, -1):
            part.append(0 if news[k] == 1 else st)
            if news[k] != 1:
                st *= news[k]
        out.extend(reversed(part))
        oi, ni = o_end, n_end
    return out if oi == len(olds) else None


def _fuse_sigmoid(ops, n_in, consts):
    """reciprocal(exp(-x) + 1) -> sig(x) inside a fused flex program: the reference's flex
    transformer does the same rewrite on the graph (FlexFusion,
    ngraph/transformers/passes/flexfusion.py: sigmoid -> SigmoidAtomicOp).  The intermediate
    registers stay defined; the compiler drops them when nothing else reads them."""
    base = n_in + len(consts)

    def producer(r):
        return ops[r - base] if r >= base else None

    def is_one(r):
        return n_in <= r < base and consts[r - n_in] == 1.0
    out = list(ops)
    for i, (name, a, b) in enumerate(ops):
        if name != "rcp":
            continue
        add = producer(a)
        if not add or add[0] != "add":
            continue
        e = add[1] if is_one(add[2]) else add[2] if is_one(add[1]) else None
        ex = producer(e) if e is not None else None
        if not ex or ex[0] != "exp":
            continue
        ng_ = producer(ex[1])
        if not ng_ or ng_[0] != "neg":
            continue
        out[i] = ("sig", ng_[1], None)
    return out


# ---------------------------------------------------------------------------------------------
class B200Transformer(object):
    """Transformer for one B200 (ngraph/transformers/gputransform.py:1034-1148 and
    flexgputransform.py:67-157 are the reference classes whose job this takes)."""

    transformer_name = "b200"
    default_rtol = 1e-05
    default_atol = 1e-08

    def __init__(self, device_id=0, flex=False, fixed_point=False, flex_verbose=False,
                 plan_only=False, fuse=True, **kwargs):
        """plan_only=True builds and compiles the kernels of every computation (NVRTC needs no
        GPU) but allocates nothing and cannot run: it exists so that the planning logic can be
        inspected and tested on a machine without a device."""
        self.plan_only = bool(plan_only)
        # fuse=False launches one kernel per op, as the reference does; in flex mode that also
        # reproduces the reference's per-op re-quantisation of every intermediate tensor
        self.fuse = bool(fuse)
        # fold bias / residual / ReLU after a convolution into the convolution step (flex16)
        self.fuse_conv_tail = bool(kwargs.pop("fuse_conv_tail", True))
        # let a kernel go on computing with a persistent tensor it has just assigned (the value
        # is taken from the register; flex16: re-quantised as the store quantises it)
        self.forward_inplace = bool(kwargs.pop("forward_inplace", True))
        self.flex = bool(flex)
        self.fixed_point = bool(fixed_point)
        self.flex_manager = flexmod.FlexManager(fixed_point=fixed_point, verbose=flex_verbose)
        self.computations = []
        self.comm = kwargs.pop("comm", None) or commmod.SingleProcessComm()
        self.bucket_bytes = int(kwargs.pop("bucket_bytes", commmod.DEFAULT_BUCKET_BYTES))
        self.min_buckets = int(kwargs.pop("min_buckets", 4))
        # random fills: the seed fixes every stream of numbers this transformer draws
        self.rng_seed = int(kwargs.pop("rng_seed", 0))
        self._rng_streams = 0
        self._alias = {}
        self._pinned = {}
        self._inputs_written = []
        self._allreduce = None      # exchange state of the computation that ran last
        self._recording = False     # a CUDA graph segment is being recorded
        self.tracer = None
        self._io_done = False       # the replayed graph has already queued the call's read-back
        self._stats_clean = False   # ... and left the statistics array cleared
        self._flex_epoch = 0        # moves whenever any exponent bookkeeping may have changed
        self._buffers = collections.OrderedDict()   # op -> Buffer
        self._views = {}
        self.finalized = False
        self.closed = False
        self._scratch_bytes = 0
        self.kernel_launches = 0
        if self.plan_only:
            return
        try:
            import torch
        except ImportError as e:    # pragma: no cover
            raise UnsupportedTransformerException("the b200 transformer needs torch: %s" % e)
        if not torch.cuda.is_available():
            raise UnsupportedTransformerException(
                "the b200 transformer needs a CUDA device; there is no CPU path")
        self.torch = torch
        self.device_id = int(device_id)
        self.device = torch.device("cuda", self.device_id)
        torch.cuda.set_device(self.device)
        self._scratch = None
        self._status = None
        self._table = None
        self._stats = None
        # TRACING=1: a Chrome-trace timeline of every launch (see tracing.py)
        self.tracer = None
        if tracing.is_tracing_enabled():
            self.tracer = tracing.TraceEventTracker(
                kwargs.pop("trace_name", "b200_trace_dev%d_%d" % (self.device_id, id(self) & 0xffff)))
            self._trace_base = torch.cuda.Event(enable_timing=True)
            self._trace_base.record(torch.cuda.current_stream(self.device))
            self._trace_calls = 0

    @property
    def stream(self):
        """Kernels go to torch's current stream (which is the capture stream while a CUDA graph
        is being recorded)."""
        return self.torch.cuda.current_stream(self.device)

    # ---- tolerances (ngraph/transformers/flexgputransform.py:80-103) ----------------------------
    def get_default_tolerance(self, desired):
        if self.flex:
            scale = flexmod.flex16.get_scale(float(np.max(np.abs(desired))))
            return scale * 8, 1e-2
        return self.default_atol, self.default_rtol

    # ---- public API ----------------------------------------------------------------------------
    def computation(self, returns, *parameters):
        if self.finalized:
            raise ValueError("Cannot create computations from a finalized transformer")
        c = Computation(self, returns, parameters)
        self.computations.append(c)
        return c

    def initialize(self):
        if self.finalized:
            return
        self.finalized = True
        for c in self.computations:
            c.build()

    def _collect_trace(self, comp, pairs):
        """After the call's synchronisation: one 'X' event per step (device time, microseconds
        since the transformer was made)."""
        self._trace_calls += 1
        for step, e0, e1 in pairs:
            self.tracer.add_operation(
                step.kind, tracing.step_name(step), self.device_id, 0,
                round(self._trace_base.elapsed_time(e0) * 1e3, 3),
                round(e0.elapsed_time(e1) * 1e3, 3),
                {"call": self._trace_calls, "step": step.index, "launches": step.launches})

    def close(self):
        if self.closed:
            return
        self.closed = True
        if getattr(self, "tracer", None) is not None and self.tracer.events:
            self.tracer.serialize_to_file()
        self._buffers.clear()
        self._views.clear()
        self._scratch = self._table = self._stats = self._status = self._probe64 = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    # ---- storage -----------------------------------------------------------------------------
    def _buffer_of(self, op):
        b = self._buffers.get(op)
        if b is None:
            persistent = isinstance(op, AssignableTensorOp)
            b = Buffer(op.name, op.axes, self.flex, persistent)
            if persistent:
                b.init_array = op.initial_array()
            if self.flex:
                b.entry = self.flex_manager.make_flex_entry(op.name)
                b.slot = self.flex_manager.new_slot()
                b.slot_write = b.slot
            self._buffers[op] = b
        return b

    def _view_of(self, op):
        while isinstance(op, SequentialOp) or op in self._alias:
            op = op.value_tensor if isinstance(op, SequentialOp) else self._alias[op]
        v = self._views.get(op)
        if v is not None:
            return v
        if isinstance(op, (BroadcastOp, ReorderAxes)):
            src = self._view_of(op.args[0])
            v = View(src.buffer, op.axes, [src.stride_of(a) for a in op.axes], src.offset)
        elif isinstance(op, AxesCastOp):
            src = self._view_of(op.args[0])
            v = View(src.buffer, op.axes, src.strides, src.offset)
        elif isinstance(op, ReshapeOp):
            src = self._view_of(op.args[0])
            strides = _reshape_strides(list(src.axes.lengths), list(src.strides),
                                       list(op.axes.lengths))
            if strides is None:
                raise ValueError("Unhandled op: {} needs a copy of its argument first "
                                 "(its elements do not lie in one regular pattern)".format(op))
            v = View(src.buffer, op.axes, strides, src.offset)
        elif isinstance(op, TensorSliceOp):
            src = self._view_of(op.args[0])
            offset = src.offset + sum(st * sr for st, sr in zip(op.starts, src.strides))
            strides = [sr * step for sr, step in zip(src.strides, op.steps) if step is not None]
            v = View(src.buffer, op.axes, strides, offset)
        elif isinstance(op, AssignOp):
            v = self._view_of(op.args[0])
        else:
            v = View.dense(self._buffer_of(op))
        self._views[op] = v
        return v

    def _write_slot(self, buf):
        if buf.persistent and buf.slot_write == buf.slot:
            buf.slot_write = self.flex_manager.new_slot()
        if buf.persistent:
            return buf.slot_write
        return buf.slot

    def _next_rng_stream(self):
        self._rng_streams += 1
        return self._rng_streams

    def _need_scratch(self, nbytes):
        self._scratch_bytes = max(self._scratch_bytes, int(nbytes))

    def _scratch_aligned(self):
        """(pointer, bytes) of the scratch arena rounded up to a 1024-byte boundary (the tensor
        core kernels place TMA-swizzled operand planes in it)."""
        base = self._scratch.data_ptr()
        off = (-base) % 1024
        return base + off, self._scratch.numel() - off

    def _slot_for_read(self, buf, step):
        if id(buf) in getattr(step, "reads_after_write", ()):
            return buf.slot_write
        return buf.slot

    def _share_entry(self, buf, src):
        """buf's values are stored with src's exponent (pooling / dimshuffle outputs)."""
        buf.entry = src.entry
        buf.slot = src.slot
        buf.slot_write = src.slot_write
        buf.shares_entry = True

    def _allocate(self, comp=None):
        if self.plan_only:
            return
        torch = self.torch
        if comp is not None and comp._comm_steps and comp._allreduce is None:
            # every tensor this computation exchanges lives in one flat fp32 arena of its own,
            # bucketed in the order the tensors are produced (step indices are per computation)
            steps = sorted(comp._comm_steps, key=lambda s: s.index)
            plan = commmod.BucketPlan([(s.key, s.arena_buffer.size) for s in steps],
                                      self.bucket_bytes, min_buckets=self.min_buckets)
            arena = torch.zeros((max(plan.total, 1),), dtype=torch.float32, device=self.device)
            funcs = {}
            last_of_bucket = {}
            for s in steps:
                off = plan.offsets[s.key]
                s.arena_buffer.tensor = arena[off:off + max(s.arena_buffer.size, 1)]
                funcs[s.key] = s.reduce_func
                last_of_bucket[plan.bucket_of[s.key]] = s
            for b_index, s in last_of_bucket.items():
                s.closes_bucket = b_index
            comp._allreduce = commmod.BucketedAllReduce(self.comm, plan, arena, funcs)
            self._allreduce = comp._allreduce
        for op, b in self._buffers.items():
            if b.tensor is None:
                dt = torch.int16 if b.flex else torch.float32
                b.tensor = torch.zeros((max(b.size, 1),), dtype=dt, device=self.device)
        for op, b in self._buffers.items():
            if b.plane_bytes > 0 and b.planes is None:
                b.planes = torch.zeros((2 * b.plane_bytes + 1024,), dtype=torch.uint8,
                                       device=self.device)
                b.planes_ptr = b.planes.data_ptr() + (-b.planes.data_ptr()) % 1024
        if self._status is None:
            self._status = torch.zeros((1,), dtype=torch.int32, device=self.device)
            self._status_host = torch.zeros((1,), dtype=torch.int32).pin_memory()
            self._probe64 = torch.zeros((1,), dtype=torch.int64, device=self.device)
        if self.flex:
            n = max(self.flex_manager.n_slots + 64, 64)
            if self._table is None or self._table.shape[0] < n:
                self._table = torch.zeros((n, 2), dtype=torch.float32, device=self.device)
                self._stats = torch.zeros((n,), dtype=torch.int32, device=self.device)
                self._table_host = torch.zeros((n, 2), dtype=torch.float32).pin_memory()
                self._stats_host = torch.zeros((n,), dtype=torch.int32).pin_memory()
                self._table_np = self._table_host.numpy()
                self._dec_uploaded = np.full((n,), -1, dtype=np.int64)   # exponent each row holds
                self._table_dirty = True
        for op, b in self._buffers.items():
            if b.init_array is not None and not getattr(b, "initialised", False):
                b.initialised = True
                self._host_to_device(View.dense(b), b.init_array, init=True)

    def _ensure_scratch(self):
        if self._scratch is None or self._scratch.numel() < self._scratch_bytes:
            self._scratch = self.torch.empty((max(self._scratch_bytes, 16) + 1024,),
                                             dtype=self.torch.uint8, device=self.device)

    # ---- host <-> device -----------------------------------------------------------------------
    def _stage(self, view, value):
        """The copy half of a host write: the fp32 values go to the device (for a flex16 tensor
        into its staging buffer).  Depends on nothing else of a call, so a computation starts
        these copies before its exponent bookkeeping."""
        torch = self.torch
        buf = view.buffer
        buf.version += 1
        if not view.is_dense():
            raise ValueError("host writes need a dense tensor")
        if isinstance(value, torch.Tensor) and value.is_cuda:
            # a tensor that already lives on the device (the reference's DeviceTensor.__setitem__
            # takes a GPUArray the same way, gputransform.py:806-854): device-to-device copy
            if tuple(value.shape) != tuple(view.axes.lengths) and \
                    tuple(value.shape) != (buf.size,):
                raise ValueError("value shape %s does not match tensor axes %s"
                                 % (tuple(value.shape), view.axes))
            src = value.to(torch.float32).reshape(-1)
            if not buf.flex:
                buf.tensor.copy_(src, non_blocking=True)
                return
            if buf.staging is None:
                buf.staging = torch.empty((max(buf.size, 1),), dtype=torch.float32,
                                          device=self.device)
            buf.staging.copy_(src, non_blocking=True)
            return
        arr = np.asarray(value, dtype=np.float32)
        # a scalar broadcasts; otherwise the shape must be the tensor's, or flat with its size
        # (a transposed or otherwise differently shaped array of the right size is an error, as
        # it is for the reference's DeviceTensor.__setitem__)
        if arr.shape not in ((), tuple(view.axes.lengths), (buf.size,)):
            squeezed = tuple(n for n in arr.shape if n != 1)
            if squeezed != tuple(n for n in view.axes.lengths if n != 1):
                raise ValueError("value shape %s does not match tensor axes %s"
                                 % (arr.shape, view.axes))
        arr = np.ascontiguousarray(np.broadcast_to(arr, view.axes.lengths)
                                   if arr.shape == () else arr.reshape(view.axes.lengths))
        src = torch.from_numpy(np.array(arr.reshape(-1), copy=not arr.flags.writeable))
        async_ok = src.is_pinned()
        if not buf.flex:
            buf.tensor.copy_(src, non_blocking=async_ok)
            return
        if buf.staging is None:
            buf.staging = torch.empty((max(buf.size, 1),), dtype=torch.float32, device=self.device)
        buf.staging.copy_(src, non_blocking=async_ok)

    def _host_to_device(self, view, value, init=False, in_call=False, staged=False):
        """DeviceTensor.__setitem__ (ngraph/transformers/gputransform.py:806-854); flex:
        FlexGPUDeviceTensor.__setitem__ (flexgputransform.py:183-208).  staged: _stage has
        already copied the values."""
        buf = view.buffer
        if not staged:
            self._stage(view, value)
        if not buf.flex:
            return
        e = buf.entry
        raw = lib.raw()
        if in_call and e.initialized:
            # exponent adopted and table row uploaded by _begin_call; the statistic is read with
            # everything else at the end of the call
            lib.check(raw.b2_flex_host_quantize(buf.staging.data_ptr(), buf.ptr(), buf.size,
                                                self._table.data_ptr(), buf.slot,
                                                self._stats.data_ptr(), self.stream.cuda_stream))
            self.kernel_launches += 1
            self._inputs_written.append(buf)
            return
        if not e.initialized:
            bits = self._stats[-1:]
            bits.zero_()
            lib.check(raw.b2_absmax_bits_f32(buf.staging.data_ptr(), buf.size, bits.data_ptr(),
                                            self.stream.cuda_stream))
            maxabs = float(bits.cpu().numpy().view(np.float32)[0])
            e.initialize_from_range(maxabs, from_host=True)
        else:
            e.begin_write()
        self._set_table_row(buf.slot, e.dec)
        self._set_table_row(buf.slot_write, e.dec)
        self._stats[buf.slot:buf.slot + 1].zero_()
        lib.check(raw.b2_flex_host_quantize(buf.staging.data_ptr(), buf.ptr(), buf.size,
                                            self._table.data_ptr(), buf.slot,
                                            self._stats.data_ptr(), self.stream.cuda_stream))
        self.kernel_launches += 1
        e.end_write(int(self._stats[buf.slot].item()))

    def _device_to_host_async(self, view):
        """Starts the device->host copy of a result into a pinned buffer; see _finish_host."""
        buf = view.buffer
        if self._allreduce is not None and getattr(buf, "comm_key", None) is not None:
            self._allreduce.wait_for(buf.comm_key)
        key = (id(buf), view.key())
        pinned = self._pinned.get(key)
        if view.is_dense():
            src = buf.tensor[:max(buf.size, 1)]
        else:
            src = self._contiguous_copy(view)
        if pinned is None:
            pinned = self.torch.empty(src.shape, dtype=src.dtype).pin_memory()
            self._pinned[key] = pinned
        pinned.copy_(src, non_blocking=True)
        return pinned, view

    def _contiguous_copy(self, view):
        """A dense device tensor holding the elements of a strided view (GPUDeviceTensor.
        as_contiguous, ngraph/transformers/gputransform.py:873-892: the same copy kernel that
        runs dimshuffles)."""
        buf = view.buffer
        lengths = list(view.axes.lengths)
        out = self.torch.empty(lengths or [1], dtype=buf.tensor.dtype, device=self.device)
        dense, acc = [], 1
        for n in reversed(lengths):
            dense.append(acc)
            acc *= n
        esize = 2 if buf.flex else 4
        lib.dimshuffle(buf.ptr() + view.offset * esize, out.data_ptr(), esize, lengths,
                       list(view.strides), list(reversed(dense)), self.stream.cuda_stream)
        self.kernel_launches += 1
        return out.reshape(lengths) if lengths else out.reshape(())

    def _finish_host(self, pending):
        """After the stream has been synchronised: a caller-owned array from the pinned copy
        (DeviceTensor.get, gputransform.py:710-744; flex: int16 * scale,
        flexgputransform.py:178-181)."""
        pinned, view = pending
        host = pinned.numpy().reshape(view.axes.lengths)
        if view.buffer.flex:
            return host.astype(np.float64) * view.buffer.entry.scale
        host = host.copy()
        if host.shape == ():
            return host[()]
        return host

    def _device_to_host(self, view):
        """DeviceTensor.get (gputransform.py:710-744); flex: int16 * scale
        (flexgputransform.py:178-181)."""
        buf = view.buffer
        flat = buf.tensor
        if self._allreduce is not None and getattr(buf, "comm_key", None) is not None:
            self._allreduce.wait_for(buf.comm_key)
        if view.is_dense():
            host = flat.cpu().numpy().reshape(view.axes.lengths)
        else:
            host = self._contiguous_copy(view).cpu().numpy()
        if buf.flex:
            return host.astype(np.float64) * buf.entry.scale
        if host.shape == ():
            return host[()]
        return host

    # ---- tensors outside computations ---------------------------------------------------------
    def device_tensor(self, op):
        """The DeviceTensor of an op's value (a variable, a placeholder, a result some
        computation keeps).  The transformer must have been initialised."""
        if self.plan_only:
            raise lib.B200Error("a plan_only transformer holds no tensors")
        if not self.finalized:
            self.initialize()
        v = self._view_of(as_op(op))
        if v.buffer.tensor is None:
            raise ValueError("no computation of this transformer uses %r" % (op,))
        return DeviceTensor(self, v)

    def get_tensor_view_value(self, op, host_tensor=None):
        """ngraph/transformers/base.py:546-558."""
        return self.device_tensor(op).get(host_tensor)

    def _write_view(self, view, value):
        """Host -> a (possibly strided) window of a tensor.  A dense whole-tensor write is the
        ordinary host write; anything else goes through a contiguous device copy of the window
        and the strided copy kernel (GPUDeviceTensor.from_other, gputransform.py:894-909)."""
        torch = self.torch
        buf = view.buffer
        lengths = list(view.axes.lengths)
        if view.is_dense():
            self._host_to_device(view, value)
            self.stream.synchronize()
            return
        arr = np.asarray(value, dtype=np.float32)
        if arr.shape not in ((), (1,)) and tuple(n for n in arr.shape if n != 1) != \
                tuple(n for n in lengths if n != 1):
            raise ValueError("value shape %s does not match the window %s" % (arr.shape, lengths))
        count = int(np.prod(lengths)) if lengths else 1
        scalar = arr.size == 1
        src = torch.from_numpy(np.ascontiguousarray(arr).reshape(-1).copy()).to(self.device)
        esize = 4
        if buf.flex:
            # FlexGPUDeviceTensor.__setitem__ (value / scale, clip, truncate)
            # A window keeps the exponent the rest of the tensor is stored with (adopting a new
            # one here would re-scale every mantissa that is not rewritten); values beyond its
            # range saturate, as FlexGPUDeviceTensor.__setitem__ clips them.
            e = buf.entry
            if not e.initialized:
                e.initialize_from_range(float(np.max(np.abs(arr))) if arr.size else 0.0,
                                        from_host=True)
            self._set_table_row(buf.slot, e.dec)
            self._set_table_row(buf.slot_write, e.dec)
            self._stats[buf.slot:buf.slot + 1].zero_()
            q = torch.empty((src.numel(),), dtype=torch.int16, device=self.device)
            lib.check(lib.raw().b2_flex_host_quantize(src.data_ptr(), q.data_ptr(), src.numel(),
                                                      self._table.data_ptr(), buf.slot,
                                                      self._stats.data_ptr(),
                                                      self.stream.cuda_stream))
            self.kernel_launches += 1
            src, esize = q, 2
        dense, acc = [], 1
        for n in reversed(lengths):
            dense.append(acc)
            acc *= n
        src_strides = [0] * len(lengths) if scalar else list(reversed(dense))
        if count:
            lib.dimshuffle(src.data_ptr(), buf.ptr() + view.offset * esize, esize, lengths,
                           src_strides, list(view.strides), self.stream.cuda_stream)
            self.kernel_launches += 1
        self.stream.synchronize()
        buf.version += 1

    # ---- flex bookkeeping ------------------------------------------------------------------------
    def _set_table_row(self, slot, dec):
        self._flex_epoch += 1
        self._stats_clean = False
        self._dec_uploaded[slot] = dec
        self._table_np[slot, 0] = 2.0 ** -dec
        self._table_np[slot, 1] = 2.0 ** dec
        self._table[slot].copy_(self._table_host[slot])

    def _set_table_row_host(self, slot, dec):
        """Updates the pinned copy of a table row; the device copy follows in one transfer."""
        if self._dec_uploaded[slot] != dec:
            self._flex_epoch += 1
            self._dec_uploaded[slot] = dec
            self._table_np[slot, 0] = math.ldexp(1.0, -dec)
            self._table_np[slot, 1] = math.ldexp(1.0, dec)
            self._table_dirty = True

    def _set_table_rows_host(self, slots, decs):
        """_set_table_row_host for arrays of rows and exponents."""
        changed = self._dec_uploaded[slots] != decs
        if changed.any():
            rows, d = slots[changed], decs[changed]
            self._flex_epoch += 1
            self._dec_uploaded[rows] = d
            self._table_np[rows, 0] = np.ldexp(1.0, (-d).astype(np.int32))
            self._table_np[rows, 1] = np.ldexp(1.0, d.astype(np.int32))
            self._table_dirty = True

    def _begin_call(self, comp):
        self._ensure_scratch()
        self._allreduce = comp._allreduce
        if self._allreduce is not None:
            self._allreduce.begin_call()
        if self.flex:
            self._begin_call_flex(comp)

    def _begin_call_flex(self, comp):
        """Exponent bookkeeping before a call (manage_before_computation of every tensor the call
        writes, flexgputransform.py:347-358): host work only, plus the upload of the scale table
        when a row changed."""
        self.flex_manager.autoflex_count += 1
        self._inputs_written = []
        steady = getattr(comp, "_steady", None)
        if steady is not None and steady[0] == self._flex_epoch and not self._table_dirty:
            # Steady state: the previous call of this computation left every exponent where it
            # was and nothing has touched the bookkeeping since, so no row of the table can move.
            if self._stats_clean:
                self._stats_clean = False
            else:
                self._stats.zero_()
            return
        comp._steady = None
        # Only tensors this computation writes (or receives from the host) can adopt a new exponent
        # here; every other tensor's table rows were brought up to date by the call that wrote it.
        bufs = getattr(comp, "_flex_bufs", None)
        if bufs is None:
            seen, bufs = set(), []
            for b in list(comp.written) + list(comp.param_buffers):
                if id(b) in seen or b.entry is None or getattr(b, "shares_entry", False):
                    continue
                seen.add(id(b))
                bufs.append(b)
            comp._flex_bufs = bufs
            for b in self._buffers.values():          # first call: every row the steps may read
                if b.entry is not None and not getattr(b, "shares_entry", False) and id(b) not in seen:
                    self._set_table_row_host(b.slot, b.entry.dec)
                    self._set_table_row_host(b.slot_write, b.entry.dec)
        if bufs:
            arrays = getattr(comp, "_flex_buf_arrays", None)
            if arrays is None:
                arrays = (np.array([b.entry.i for b in bufs], dtype=np.int64),
                          np.array([b.slot_write for b in bufs], dtype=np.int64),
                          np.array([b.slot for b in bufs], dtype=np.int64))
                comp._flex_buf_arrays = arrays
            ids, slot_w, slot_r = arrays
            fm = self.flex_manager
            dec_stored = fm.dec[ids].copy()
            # tensors this call overwrites adopt the exponent chosen after their previous write
            dec_w = dec_stored.copy()
            init = fm.initialized[ids]
            if init.any():
                dec_w[init] = fm.begin_write_batch(ids[init])
            self._set_table_rows_host(slot_w, dec_w)
            two = slot_r != slot_w
            if two.any():
                self._set_table_rows_host(slot_r[two], dec_stored[two])
        if self._table_dirty:
            self._table.copy_(self._table_host, non_blocking=True)
            self._table_dirty = False
        if self._stats_clean:
            self._stats_clean = False
        else:
            self._stats.zero_()

    def _publish(self):
        """Status word and flex statistics into pinned host memory, statistics cleared: one
        small launch (lib: b2_flex_publish)."""
        n = self._stats.numel() if self.flex else 0
        lib.check(lib.raw().b2_flex_publish(
            self._stats.data_ptr() if self.flex else None, n, self._status.data_ptr(),
            self._stats_host.data_ptr() if self.flex else None, self._status_host.data_ptr(),
            self.stream.cuda_stream))
        self.kernel_launches += 1

    def _end_call(self, comp):
        """One synchronisation per call: statistics and status come back together."""
        torch = self.torch
        if self._io_done:
            self._io_done = False          # the replayed graph ended with the read-back
        else:
            self._publish()
            self._stats_clean = self.flex
        exchanging = self._allreduce is not None and self.comm.size > 1
        if exchanging:
            self._allreduce.finish()        # CommError instead of an endless synchronisation
        torch.cuda.current_stream(self.device).synchronize()
        if exchanging:
            self._allreduce.after_sync()
        for b in comp.written:
            b.version += 1
        if int(self._status_host[0]) != 0:
            self._status.zero_()
            raise lib.B200Error("a device-side wait ran out during the computation")
        if self.flex:
            self._end_call_flex(comp)

    def _end_call_flex(self, comp):
        """Exponent bookkeeping after a call (manage_after_computation, flexgputransform.py:
        360-366) from the statistics the call left in pinned host memory."""
        stats = self._stats_host.numpy()
        steady = getattr(comp, "_steady", None)
        if steady is not None and steady[0] == self._flex_epoch and \
                len(self._inputs_written) == steady[3] and np.array_equal(stats[steady[1]], steady[2]):
            # the same maxima as after the previous call, with every history window already full
            # of them: every entry would make the choice it made before
            return
        self._flex_epoch += 1
        fm = self.flex_manager
        for b in self._inputs_written:
            b.entry.end_write(int(stats[b.slot]))
        arrays = getattr(comp, "_flex_written_arrays", None)
        if arrays is None:
            ids = np.array([b.entry.i for b in comp.written], dtype=np.int64)
            arrays = (ids, np.array([b.slot_write for b in comp.written], dtype=np.int64),
                      len(set(ids.tolist())) == len(ids))
            comp._flex_written_arrays = arrays
        ids, slots, distinct = arrays
        if distinct:
            fm.end_write_batch(ids, stats[slots])      # all written tensors in a few array ops
        else:
            for b in comp.written:                     # an entry written twice: one at a time
                b.entry.end_write(int(stats[b.slot_write]))
        in_ids = np.array([b.entry.i for b in self._inputs_written], dtype=np.int64)
        if fm.settled(ids) and fm.settled(in_ids):
            idx = np.concatenate([np.array([b.slot for b in self._inputs_written], dtype=np.int64),
                                  slots])
            comp._steady = (self._flex_epoch, idx, stats[idx].copy(), len(self._inputs_written))
        else:
            comp._steady = None

    # ---- launching -------------------------------------------------------------------------------
    def _launch_step(self, step):
        if self._allreduce is not None and not self._recording:
            for v in step.in_views:
                key = getattr(v.buffer, "comm_key", None)
                if key is not None and step.kind != "comm":
                    self._allreduce.wait_for(key)      # first consumer of a reduced tensor
        if step.kind == "ew":
            self._launch_ew(step)
        else:
            step.launch(self)

    def _launch_ew(self, step):
        ins = [v.buffer.ptr() + v.offset * (2 if v.buffer.flex else 4) for v in step.in_views]
        outs = [v.buffer.planes_ptr if as_planes else
                v.buffer.ptr() + v.offset * (2 if v.buffer.flex else 4)
                for v, as_planes in step.out_targets]
        common = dict(consts=step.consts, scratch=self._scratch.data_ptr(),
                      scratch_bytes=self._scratch.numel(), status=self._status.data_ptr(),
                      stream=self.stream.cuda_stream)
        if self.flex:
            common.update(flex_table=self._table.data_ptr(), flex_stats=self._stats.data_ptr())
            fresh = [b for b in step.output_buffers() if not b.entry.initialized]
            # First write of these tensors: measure the unsaturated range, then pick exponents.
            # The measuring launch leaves float bits in the statistic of EVERY output of the
            # kernel, so the statistics of the outputs that are not new are put back after it.
            # A new tensor whose value depends on the STORED form of another new tensor of the
            # same kernel (a requant op) is measured in a later round, once that exponent exists.
            deps = getattr(step, "requant_deps", None) or [0] * len(step.out_targets)
            while fresh:
                saved = self._stats.clone()
                # bit k: result k has no exponent yet (a requant op on it passes values through)
                open_bits = sum(1 << k for k, (v, _) in enumerate(step.out_targets)
                                if v.buffer in fresh)
                step.kernel.launch(ins, outs, probe=1 | (open_bits << 1), **common)
                self.kernel_launches += step.kernel.launches
                self._stats_host.copy_(self._stats, non_blocking=False)
                self._stats.copy_(saved)
                bits = self._stats_host.numpy()
                ready = [b for b in fresh
                         if not any(v.buffer is b and (deps[k] & open_bits & ~(1 << k))
                                    for k, (v, _) in enumerate(step.out_targets))]
                if not ready:            # cannot happen (ops are ordered); do not loop for ever
                    ready = list(fresh)
                for b in ready:
                    maxabs = float(bits[b.slot_write:b.slot_write + 1].view(np.float32)[0])
                    dec = b.entry.initialize_from_range(maxabs)
                    self._set_table_row(b.slot_write, dec)
                    self._stats[b.slot_write:b.slot_write + 1].zero_()
                fresh = [b for b in fresh if b not in ready]
        step.kernel.launch(ins, outs, **common)
        self.kernel_launches += step.kernel.launches


class DeviceTensor(object):
    """A tensor (or a window of one) on the device, readable and writable from the host outside
    any computation: GPUDeviceTensor.get / __getitem__ / __setitem__
    (ngraph/transformers/gputransform.py:679-909) and, for flex16 storage, FlexGPUDeviceTensor
    (ngraph/transformers/flexgputransform.py:160-208): values are read as mantissa * scale and
    written as value / scale, clipped to the int16 range and truncated, with the tensor's
    exponent entry told the largest magnitude written.

        w = transformer.device_tensor(variable)
        w.get()                      # numpy copy of the whole tensor
        w[2:5, :, 0].get()           # a window: slices and integers per axis, Ellipsis
        w[...] = array               # whole tensor; w[1:3] = 0.5 fills a window
    """

    def __init__(self, transformer, view):
        self.transformer = transformer
        self.view = view

    @property
    def shape(self):
        return tuple(self.view.axes.lengths)

    @property
    def scale(self):
        e = self.view.buffer.entry
        return e.scale if e is not None else 1.0

    def get(self, tensor=None):
        host = self.transformer._device_to_host(self.view)
        if tensor is None:
            return host
        tensor[...] = host
        return tensor

    def __getitem__(self, index):
        if index is None or index is Ellipsis or index == ():
            return self
        if not isinstance(index, tuple):
            index = (index,)
        v = self.view
        n = len(v.axes)
        if Ellipsis in index:
            k = index.index(Ellipsis)
            fill = n - (len(index) - 1)
            if fill < 0 or Ellipsis in index[k + 1:]:
                raise IndexError("too many indices for a tensor of %d axes" % n)
            index = index[:k] + (slice(None),) * fill + index[k + 1:]
        if len(index) > n:
            raise IndexError("too many indices for a tensor of %d axes" % n)
        index = index + (slice(None),) * (n - len(index))
        axes, strides, offset = [], [], v.offset
        for a, st, ix in zip(v.axes, v.strides, index):
            if isinstance(ix, slice):
                start, stop, step = ix.indices(a.length)
                if step <= 0:
                    raise IndexError("slices of device tensors need a positive step")
                count = max(0, -(-(stop - start) // step))
                offset += start * st
                axes.append(a if count == a.length else type(a)(count, a.name))
                strides.append(st * step)
            else:
                i = int(ix)
                if i < 0:
                    i += a.length
                if not 0 <= i < a.length:
                    raise IndexError("index %d is out of bounds for axis %s" % (ix, a))
                offset += i * st
        return DeviceTensor(self.transformer, View(v.buffer, axes, strides, offset))

    def __setitem__(self, key, value):
        self.transformer._write_view(self.__getitem__(key).view, value)


# ---------------------------------------------------------------------------------------------
# registry / factories (ngraph/transformers/base.py:265-279, 807-847)
# ---------------------------------------------------------------------------------------------
_transformers = {B200Transformer.transformer_name: B200Transformer}
_factory = None


def transformer_choices():
    return sorted(_transformers.keys())


def allocate_transformer(name, **kwargs):
    try:
        cls = _transformers[name]
    except KeyError:
        raise ValueError("The given transformer name ({}) is invalid/unsupported.".format(name))
    return cls(**kwargs)


def make_transformer_factory(name, **kwargs):
    def factory():
        return allocate_transformer(name, **kwargs)
    factory.name = name
    return factory


def set_transformer_factory(factory):
    global _factory
    _factory = factory


def make_transformer():
    f = _factory or make_transformer_factory("b200")
    return f()
