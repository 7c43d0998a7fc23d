"""Layout and fusion: turns elementwise / reduction / assign ops into fused kernel programs.

Takes the place of the reference's GPU layout pass and of the (never enabled) elementwise fusion
its kernel generator was written for:
  * ngraph/transformers/passes/layout.py:104-339 + gpu/gpulayout.py: the reference only ever
    picks each op's default layout, so here every tensor is stored dense in its op's axis order
    and views (broadcast / reorder) become stride descriptors;
  * ngraph/transformers/gputransform.py:86-108 (`ElementWiseKernel.ops_buffer`) and
    gpu/float_ew2.py:553-612 (`_preprocess_ops`): maximal connected sets of elementwise ops that
    share an iteration space, plus the reductions that consume them, become ONE kernel.

Ordering rule (reference: Op.ordered_ops sorts over args and control deps,
ngraph/op_graph/op_graph.py:245-299): steps run in creation order; an op may join an existing
group only if everything it depends on -- including earlier in-place writes to a tensor it reads,
and earlier reads of a tensor it overwrites -- belongs to a step that is not later than that
group.
"""
from . import lib
from .op_graph import (AssignableTensorOp, AssignOp, ElementWiseOp, ReductionOp)

MAX_IN = lib.EW_MAX_IN - 1
MAX_OUT = lib.EW_MAX_OUT
MAX_OPS = lib.EW_MAX_OPS - 8
MAX_CONST = lib.EW_MAX_CONST


class EwGroup(object):
    """One fused kernel under construction."""

    def __init__(self, index, iter_axes):
        self.index = index
        self.iter_axes = iter_axes
        self.red_axes = None
        self.members = []          # ops in execution order (ElementWiseOp / ReductionOp / AssignOp)
        self.member_set = set()
        self.ext_inputs = []       # distinct external loads (views)
        self.after_write = {}      # view key -> read happens after an in-place write
        self.n_consts = 0
        self.stored = set()        # members known to need a store (returned, reduced, consumed outside)

    kind = "ew"

    def has(self, op):
        return op in self.member_set

    def add(self, op):
        self.members.append(op)
        self.member_set.add(op)

    def __repr__(self):
        return "<EwGroup %d %s %d ops>" % (self.index, self.iter_axes, len(self.members))


def collapse_dims(lengths, strides_list, reduced):
    """Merges adjacent iteration axes that every tensor walks contiguously.

    lengths: extents of the iteration axes (outermost first); strides_list: per tensor, the
    element stride along each axis (0 = broadcast); reduced: per axis, True if reduced.
    Returns (lengths, strides_list, reduced) with length-1 axes dropped and mergeable neighbours
    merged.  (The reference flattens to at most three axes the same way,
    ngraph/transformers/gpu/float_ew2.py:285-286,426-550.)
    """
    keep = [i for i, n in enumerate(lengths) if n != 1]
    lengths = [lengths[i] for i in keep]
    strides_list = [[s[i] for i in keep] for s in strides_list]
    reduced = [reduced[i] for i in keep]
    i = 0
    while i + 1 < len(lengths):
        ok = reduced[i] == reduced[i + 1]
        if ok:
            for s in strides_list:
                if s[i] != s[i + 1] * lengths[i + 1]:
                    ok = False
                    break
        if ok:
            lengths[i:i + 2] = [lengths[i] * lengths[i + 1]]
            reduced[i:i + 2] = [reduced[i]]
            for s in strides_list:
                s[i:i + 2] = [s[i + 1]]
        else:
            i += 1
    return lengths, strides_list, reduced


def map_to_abc(lengths, strides_list, reduced):
    """Places collapsed axes on the kernel's [A, B, C] space; returns
    (dims, strides_list (sa, sb, sc), reduce_mode) or raises ValueError."""
    n = len(lengths)
    nred = sum(1 for r in reduced if r)
    if nred == 0:
        if n > 3:
            raise ValueError("Unhandled op: elementwise kernel over %d non-mergeable axes" % n)
        pad = 3 - n
        dims = [1] * pad + list(lengths)
        out = [tuple([0] * pad + list(s)) for s in strides_list]
        return tuple(dims), out, lib.REDUCE_NONE
    if nred > 1:
        raise ValueError("Unhandled op: reduction over non-adjacent axes")
    r = reduced.index(True)
    if r == n - 1:                       # innermost axis reduced
        if n > 3:
            raise ValueError("Unhandled op: reduction kernel over %d non-mergeable axes" % n)
        pad = 3 - n
        dims = [1] * pad + list(lengths)
        out = [tuple([0] * pad + list(s)) for s in strides_list]
        return tuple(dims), out, lib.REDUCE_C
    # reduced axis followed by exactly one kept axis, preceded by at most one
    if n - 1 - r != 1 or r > 1:
        raise ValueError("Unhandled op: reduction axis in an unsupported position")
    if r == 0:
        dims = [1] + list(lengths)
        out = [tuple([0] + list(s)) for s in strides_list]
    else:
        dims = list(lengths)
        out = [tuple(s) for s in strides_list]
    return tuple(dims), out, lib.REDUCE_B
