"""CPU restatement of the reference's Flexpoint (flex16) arithmetic and exponent management.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this file; it exists so that
the GPU path can be checked against an independent numpy statement of the same rules.

Parity status
-------------
* quantise / saturate / de-quantise / maxabs statistic / host<->device conversion: follow the
  reference sources cited on each function ("pinned by source").
* exponent range, first-call initialisation and the overflow response: pinned by the golden
  vectors in the reference's tests/flex_tests (transcribed in tests/golden/flex_vectors.py).
* the history predictor (`Autoflex.predict_dec`): the reference delegates it to the external,
  un-vendored `autoflex` package (ngraph/flex/__init__.py:1-4, no version pinned).  The rule here
  (max of the last 16 observed maxima + 3 population standard deviations) is a restatement of the
  published Flexpoint exponent-prediction scheme fitted to every multi-call golden vector; beyond
  those vectors it is PARITY UNPINNED.
"""
from collections import deque

import numpy as np

F32 = np.float32
MANT_MAX = 32767           # dtype.pclip  (ngraph/transformers/flexgputransform.py:191-195)
MANT_MIN = -32768          # dtype.nclip
DEC_MIN = 0                # 5 exponent bits: ngraph/flex/base.py:24
DEC_MAX = 31
DEFAULT_DEC = 8            # ngraph/flex/base.py:89
HISTORY = 16


def scale_of(dec):
    """scale = 2**-dec (ngraph/flex/base.py:63-75)."""
    return 2.0 ** (-int(dec))


def dequantize(mant, dec):
    """`scale_in * (float)int16` in fp32 (ngraph/transformers/gpu/float_ew2.py:96)."""
    return np.asarray(mant).astype(F32) * F32(scale_of(dec))


def quantize(val, dec):
    """Device store: cvt.rni.s16.f32(val * (1/scale)) -- fp32 multiply, round to nearest even,
    saturate to [-32768, 32767], NaN -> 0 (ngraph/transformers/gpu/float_ew2.py:97,261-267)."""
    with np.errstate(all="ignore"):
        t = np.asarray(val, dtype=F32) * F32(2.0 ** int(dec))
        r = np.rint(t)
        r = np.where(np.isnan(r), F32(0), r)
        return np.clip(r, MANT_MIN, MANT_MAX).astype(np.int16)


def maxabs_stat(mant):
    """max |mantissa| as s32, so -32768 counts as 32768
    (ngraph/transformers/gpu/float_ew2.py:269-281)."""
    m = np.asarray(mant).astype(np.int32)
    return int(np.max(np.abs(m))) if m.size else 0


def host_to_mantissa(value, dec):
    """Host write: value / scale, clip to [-2^15, 2^15-1], numpy float->int16 assignment
    (truncation toward zero); returns (mantissas, maxabs)
    (ngraph/transformers/flexgputransform.py:183-208, gputransform.py:806-838)."""
    v = np.asarray(value, dtype=np.float64) / scale_of(dec)
    v = np.clip(v, MANT_MIN, MANT_MAX)
    maxabs = int(np.max(np.abs(v))) if v.size else 0
    return np.trunc(v).astype(np.int16), maxabs


def mantissa_to_host(mant, dec):
    """Device read: int16 * scale (ngraph/transformers/flexgputransform.py:178-181)."""
    return np.asarray(mant).astype(np.float64) * scale_of(dec)


def fit_dec(maxabs_real):
    """Largest dec in [0, 31] with maxabs_real * 2**dec <= 32767 (golden vectors:
    tests/flex_tests/test_flexew/test_complex_math.py:33-36,47-50,100-109)."""
    a = float(maxabs_real)
    if not np.isfinite(a):
        return DEC_MIN
    if a <= 0.0:
        return None
    dec = int(np.floor(np.log2(MANT_MAX / a)))
    # guard the floating log at exact powers of two
    while dec < DEC_MAX and a * 2.0 ** (dec + 1) <= MANT_MAX:
        dec += 1
    while dec > DEC_MIN and a * 2.0 ** dec > MANT_MAX:
        dec -= 1
    return int(min(max(dec, DEC_MIN), DEC_MAX))


class FlexEntry(object):
    """Per-buffer exponent state (interface of ngraph/flex/base.py:47-75 plus the history the
    external manager keeps)."""

    def __init__(self, name="", fixed_point=False):
        self.name = name
        self.dec = DEFAULT_DEC
        self.fixed_point = fixed_point
        self.initialized = fixed_point
        self.history = deque(maxlen=HISTORY)   # observed real-valued maxima
        self.next_dec = None                   # chosen by observe(), applied by prepare_write()

    @property
    def scale(self):
        return scale_of(self.dec)

    def reset(self):
        self.__init__(self.name, self.fixed_point)

    # -- first observation ------------------------------------------------------------------
    def initialize(self, maxabs_real):
        """Choose the exponent for a tensor never written before from the true (unsaturated)
        maximum of what is about to be written.  A zero maximum keeps the default dec 8
        (tests/flex_tests/test_flexew/test_flexew_inequalities.py:49-55: operand 1 first holds 0,
        then -32768 is stored as -128)."""
        if self.fixed_point:
            return
        d = fit_dec(maxabs_real)
        if d is not None:
            self.dec = d
        self.initialized = True

    # -- before every write after the first ---------------------------------------------------
    def prepare_write(self):
        """manage_before_computation: the exponent chosen from the previous observations takes
        effect when the tensor is about to be overwritten (flexgputransform.py:347-358)."""
        if self.next_dec is not None:
            self.dec = self.next_dec
            self.next_dec = None

    # -- after every write ------------------------------------------------------------------
    def observe(self, maxabs_mant):
        """manage_after_computation: record the integer maxabs of one write and choose the
        exponent for the next write (flexgputransform.py:360-366)."""
        if self.fixed_point:
            return
        if maxabs_mant >= MANT_MAX:
            # saturation: the true maximum is unknown.  Next write gets 4x the range; the
            # history remembers twice the saturated value.
            self.history.append(2.0 * maxabs_mant * self.scale)
            self.next_dec = max(self.dec - 2, DEC_MIN)
            return
        self.history.append(maxabs_mant * self.scale)
        self.next_dec = predict_dec(self.history)


def predict_dec(history):
    """Exponent for the next write from the recent maxima: the largest dec that still holds
    max(history) + 3 * std(history) (population std)."""
    h = np.asarray(history, dtype=np.float64)
    if h.size == 0:
        return None
    pred = float(h.max() + 3.0 * h.std())
    return fit_dec(pred)
