"""Drives the CPU flex oracle through the same call sequences as the reference's flex test
templates (ngraph/testing/flex_util.py:114-160): placeholders are written from the host, every
graph op is one flex kernel, the result is read back as a float."""
import numpy as np

from oracle import ew_oracle as ew
from oracle import flex_oracle as fx

REDUCTIONS = ("sum", "prod", "max", "min", "argmax", "argmin")


class FlexSimExecutor(object):
    def __init__(self, op, n_operands, fixed_point=False):
        self.op = op
        self.ph = [ew.FlexTensor("ph%d" % i, fixed_point) for i in range(n_operands)]
        self.tmp = {}
        self.fixed_point = fixed_point

    def _t(self, name):
        if name not in self.tmp:
            self.tmp[name] = ew.FlexTensor(name, self.fixed_point)
        return self.tmp[name]

    def __call__(self, *operands):
        for t, v in zip(self.ph, operands):
            t.host_write(v)
        op = self.op
        if op == "assign_var":
            out = ew.flex_kernel("assign", self._t("v"), self.ph[0])
        elif op == "sigmoid_composed":
            # reciprocal(exp(-x) + 1)  (ngraph/op_graph/op_graph.py:4198)
            one = self._t("one")
            if one.mant is None:
                one.host_write(1.0)
            n = ew.flex_kernel("neg", self._t("neg"), self.ph[0])
            e = ew.flex_kernel("exp", self._t("exp"), n)
            a = ew.flex_kernel("add", self._t("add"), e, one)
            out = ew.flex_kernel("rcp", self._t("rcp"), a)
        elif op in REDUCTIONS:
            out = ew.flex_kernel(op, self._t("out"), self.ph[0], axis=None)
        else:
            out = ew.flex_kernel(op, self._t("out"), *self.ph)
        return out.host_read()


def flex_tolerance(desired):
    """FlexGPUTransformer.get_default_tolerance (flexgputransform.py:98-103); the scale of the
    expected maximum is the one the exponent manager would give a tensor holding it."""
    m = float(np.max(np.abs(desired)))
    d = fx.fit_dec(m)
    scale = fx.scale_of(d if d is not None else fx.DEFAULT_DEC)
    return 8 * scale, 1e-2
