"""Evaluates a graph of ngraph_python_b200 ops with numpy (fp32), using the oracle's op
semantics.  Test infrastructure: it lets the graph-building surface (axes, broadcasting by axis
name, dot contraction, views, sequential/assign ordering) and the reference->mirror translation
be checked against the reference CPU transformer's fixtures on a machine without a GPU.  The
product has no such path."""
import numpy as np

from ngraph_python_b200 import op_graph as g
from oracle import conv_oracle as co
from oracle import lut_oracle as lo
from oracle import ew_oracle as ew


class Interp(object):
    def __init__(self, allreduce=None):
        """allreduce(array, reduce_func) -> array: what an AllReduceOp does (identity when None,
        i.e. one replica); a multi-process test passes a gloo collective here."""
        self.state = {}      # AssignableTensorOp -> ndarray (axes order of the op)
        self.cache = {}
        self.allreduce = allreduce

    def _to(self, val, src_axes, dst_axes):
        """Re-lay `val` (axes src_axes) out over dst_axes (superset, any order), broadcasting."""
        src = list(src_axes)
        dst = list(dst_axes)
        perm = [src.index(a) for a in dst if a in src]
        v = np.transpose(val, perm) if perm else val
        shape = [a.length if a in src else 1 for a in dst]
        return np.broadcast_to(v.reshape(shape), [a.length for a in dst])

    def run(self, outs, feeds):
        self.cache = {}
        for op, v in feeds.items():
            self.state[op] = np.asarray(v, dtype=np.float32).reshape(op.axes.lengths)
        return [np.array(self.eval(o), copy=True) for o in outs]

    def eval(self, op):
        if isinstance(op, g.SequentialOp):
            val = None
            for o in op.ops:
                val = self.eval(o)
            return val
        if isinstance(op, g.AssignableTensorOp):
            if op not in self.state:
                init = op.initial_array()
                self.state[op] = (np.zeros(op.axes.lengths, np.float32) if init is None
                                  else np.array(init, copy=True))
            return self.state[op]
        if isinstance(op, g.AssignOp):
            tgt, val = op.args
            new = np.array(self._to(self.eval(val), val.axes, tgt.axes), copy=True)
            if isinstance(tgt, g.TensorSliceOp):          # assignment into a slice of a tensor
                base = self.eval(tgt.args[0])             # the state array itself
                base[tgt.slices] = new.reshape(base[tgt.slices].shape)
            else:
                self.state[tgt] = new
            return None
        if op in self.cache:
            return self.cache[op]
        out = self._compute(op)
        self.cache[op] = out
        return out

    def _compute(self, op):
        if isinstance(op, (g.BroadcastOp, g.ReorderAxes)):
            return self._to(self.eval(op.args[0]), op.args[0].axes, op.axes)
        if isinstance(op, g.TensorSliceOp):
            return np.asarray(self.eval(op.args[0]))[op.slices].reshape(op.axes.lengths)
        if isinstance(op, (g.AxesCastOp, g.ReshapeOp)):
            return np.ascontiguousarray(self.eval(op.args[0])).reshape(op.axes.lengths)
        if isinstance(op, g.ElementWiseOp):
            args = [self._to(self.eval(a), a.axes, op.axes) for a in op.args]
            return ew.apply(op.opname, *args).astype(np.float32)
        if isinstance(op, g.ReductionOp):
            x = op.args[0]
            v = self._to(self.eval(x), x.axes, list(op.axes) + list(op.reduction_axes))
            flat = v.reshape([a.length for a in op.axes] + [-1])
            return ew.apply(op.redop, flat, axis=-1).reshape(op.axes.lengths)
        if isinstance(op, g.DotOp):
            x, y = op.args
            red = list(op.reduction_axes)
            xv = self._to(self.eval(x), x.axes, list(op.x_out_axes) + red)
            yv = self._to(self.eval(y), y.axes, red + list(op.y_out_axes))
            k = int(np.prod([a.length for a in red])) if red else 1
            out = xv.reshape(-1, k).astype(np.float64) @ yv.reshape(k, -1).astype(np.float64)
            return out.astype(np.float32).reshape(op.axes.lengths)
        if isinstance(op, (g.ConvolutionOp, g.bprop_conv, g.update_conv)):
            a, b = [self.eval(x) for x in op.args]
            cp = op.conv_params
            geo = [tuple(int(cp.get(k + "_" + d, dflt)) for d in "dhw")
                   for k, dflt in (("pad", 0), ("str", 1), ("dil", 1))]
            if isinstance(op, g.ConvolutionOp):
                out = co.conv3d_fprop(a, b, *geo)
            elif isinstance(op, g.bprop_conv):            # args (delta, filters)
                out = co.conv3d_bprop(a, b, op.axes.lengths[1:4], *geo)
            else:                                         # args (delta, inputs)
                out = co.conv3d_update(b, a, op.axes.lengths[1:4], *geo)
            return out.reshape(op.axes.lengths)
        if isinstance(op, g.LookupTableOp):
            lut, idx = self.eval(op.args[0]), self.eval(op.args[1])
            return lo.lut_fprop(lut, idx, op.lut_axis).reshape(op.axes.lengths)
        if isinstance(op, g.update_lut):
            delta, idx = self.eval(op.args[0]), self.eval(op.args[1])
            return lo.lut_update(delta, idx, op.pad_idx, op.lut_axis, op.axes.lengths)
        if isinstance(op, g.BpropPoolOp):
            e, i = self.eval(op.args[0]), self.eval(op.args[1])
            pp = op.pool_params
            out = co.pool_bprop(e[:, 0], i[:, 0], (pp["R"], pp["S"]), (pp["pad_h"], pp["pad_w"]),
                                (pp["str_h"], pp["str_w"]), pp["op"])
            return out[:, None].reshape(op.axes.lengths)
        if isinstance(op, g.PoolingOp):
            i = self.eval(op.args[0])
            pp = op.pool_params
            fn = co.pool_max_fprop if pp["op"] == "max" else co.pool_avg_fprop
            out = fn(i[:, 0], (pp["R"], pp["S"]), (pp["pad_h"], pp["pad_w"]),
                     (pp["str_h"], pp["str_w"]))
            return out[:, None].reshape(op.axes.lengths)
        if isinstance(op, g.AllReduceOp):
            val = self.eval(op.args[0])
            if self.allreduce is None:
                return val
            return np.asarray(self.allreduce(np.ascontiguousarray(val, dtype=np.float32),
                                             op.reduce_func), dtype=np.float32)
        raise ValueError("Unhandled op: {}".format(op))
