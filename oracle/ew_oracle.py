"""CPU restatement of the reference's elementwise / reduction op semantics (fp32 and flex16).

TEST INFRASTRUCTURE ONLY: used by tests/, the smoke check and the CPU-baseline leg of the bench.
Each op follows the CUDA-C template the reference generates for it
(ngraph/transformers/gpu/float_ew2.py:31-90): all arithmetic is fp32; transcendental functions
are evaluated in float64 and rounded once to fp32 (CUDA libm is within 1-2 ulp of that).
"""
import numpy as np

from . import flex_oracle as fx

F32 = np.float32


def _f64(fn):
    def wrapped(x):
        with np.errstate(all="ignore"):
            return fn(np.asarray(x, dtype=np.float64)).astype(F32)
    return wrapped


def _cmp(fn):
    def wrapped(x, y):
        return fn(x, y).astype(F32)
    return wrapped


def _int_mod(x, y):
    # `int(x) % int(y)`: C truncation toward zero, sign of the dividend
    xi = np.trunc(x).astype(np.int64)
    yi = np.trunc(y).astype(np.int64)
    with np.errstate(all="ignore"):
        return np.fmod(xi, np.where(yi == 0, 1, yi)).astype(F32)


def _int_div(x, y):
    xi = np.trunc(x).astype(np.int64)
    yi = np.trunc(y).astype(np.int64)
    with np.errstate(all="ignore"):
        q = np.trunc(xi / np.where(yi == 0, 1, yi))
    return q.astype(F32)


def _binary32(fn):
    def wrapped(x, y):
        with np.errstate(all="ignore"):
            return fn(np.asarray(x, F32), np.asarray(y, F32)).astype(F32)
    return wrapped


def _pow(x, y):
    with np.errstate(all="ignore"):
        return np.power(np.asarray(x, np.float64), np.asarray(y, np.float64)).astype(F32)


def _sig(x):
    # 1.0f / (1.0f + expf(-x))   (float_ew2.py:44)
    with np.errstate(all="ignore"):
        e = np.exp(-np.asarray(x, np.float64)).astype(F32)
        return (F32(1.0) / (F32(1.0) + e)).astype(F32)


UNARY = {
    "assign": lambda x: np.asarray(x, F32),
    "neg": lambda x: -np.asarray(x, F32),
    "abs": lambda x: np.abs(np.asarray(x, F32)),
    "sqrt": _f64(np.sqrt),
    "sqr": lambda x: (np.asarray(x, F32) * np.asarray(x, F32)).astype(F32),
    "exp": _f64(np.exp),
    "log": _f64(np.log),
    "safelog": lambda x: np.where(np.asarray(x, F32) > 0, _f64(np.log)(x), F32(-50.0)).astype(F32),
    "rcp": lambda x: _binary32(np.divide)(F32(1.0), x),
    "sig": _sig,
    "tanh": _f64(np.tanh),
    "sin": _f64(np.sin),
    "cos": _f64(np.cos),
    "sgn": lambda x: np.sign(np.asarray(x, F32)).astype(F32),
}

BINARY = {
    "add": _binary32(np.add),
    "sub": _binary32(np.subtract),
    "mul": _binary32(np.multiply),
    "div": _binary32(np.divide),
    "mod": _int_mod,
    "int_div": _int_div,
    "pow": _pow,
    "minimum": _binary32(np.fmin),
    "maximum": _binary32(np.fmax),
    "eq": _cmp(np.equal),
    "ne": _cmp(np.not_equal),
    "lt": _cmp(np.less),
    "le": _cmp(np.less_equal),
    "gt": _cmp(np.greater),
    "ge": _cmp(np.greater_equal),
}


def _seq_reduce(fn, init):
    """fp32 accumulation (the reduction order differs between implementations; tests allow for
    that with a tolerance on sums, exact on max/min/arg*)."""
    def wrapped(x, axis):
        x = np.asarray(x, F32)
        return fn(x, axis=axis).astype(F32)
    return wrapped


def _argmax(x, axis):
    # first index holding the maximum (strict > update, float_ew2.py:74)
    return np.argmax(np.asarray(x, F32), axis=axis).astype(F32)


def _argmin(x, axis):
    return np.argmin(np.asarray(x, F32), axis=axis).astype(F32)


REDUCE = {
    "sum": _seq_reduce(np.sum, 0.0),
    "prod": _seq_reduce(np.prod, 1.0),
    "max": _seq_reduce(np.max, None),
    "min": _seq_reduce(np.min, None),
    "argmax": _argmax,
    "argmin": _argmin,
}


def apply(op, *args, **kw):
    if op in UNARY:
        return UNARY[op](*args)
    if op in BINARY:
        return BINARY[op](*args)
    if op in REDUCE:
        return REDUCE[op](args[0], kw.get("axis", None))
    raise ValueError("Unhandled op %r" % (op,))


# ---------------------------------------------------------------------------------------------
# flex16 single-kernel model: every op is one kernel whose inputs are de-quantised, computed in
# fp32 and re-quantised with the output entry's exponent (float_ew2.py:93-98,1346-1404).
# ---------------------------------------------------------------------------------------------
class FlexTensor(object):
    def __init__(self, name="", fixed_point=False):
        self.entry = fx.FlexEntry(name, fixed_point)
        self.mant = None

    def host_write(self, value):
        """FlexGPUDeviceTensor.__setitem__ (flexgputransform.py:183-208)."""
        value = np.asarray(value, dtype=np.float64)
        e = self.entry
        if not e.initialized:
            e.initialize(float(np.max(np.abs(value))) if value.size else 0.0)
        else:
            e.prepare_write()
        self.mant, maxabs = fx.host_to_mantissa(value, e.dec)
        e.observe(maxabs)

    def kernel_write(self, val_f32):
        e = self.entry
        val_f32 = np.asarray(val_f32, F32)
        if not e.initialized:
            with np.errstate(all="ignore"):
                a = np.abs(val_f32.astype(np.float64))
                a = np.where(np.isnan(a), 0.0, a)
                e.initialize(float(a.max()) if a.size else 0.0)
        else:
            e.prepare_write()
        self.mant = fx.quantize(val_f32, e.dec)
        e.observe(fx.maxabs_stat(self.mant))

    def value(self):
        return fx.dequantize(self.mant, self.entry.dec)

    def host_read(self):
        return fx.mantissa_to_host(self.mant, self.entry.dec)


def flex_kernel(op, out, *ins, **kw):
    """One flex kernel: out <- quantise(op(de-quantise(ins)))."""
    vals = [t.value() for t in ins]
    out.kernel_write(apply(op, *vals, **kw))
    return out
