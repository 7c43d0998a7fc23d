"""Flexpoint (flex16) exponent management for the B200 transformer.

Takes the place of the reference's Flex/FlexEntry/FlexManager interface (ngraph/flex/base.py) and
of the external `autoflex.gpu.GPUFlexManager` it delegates to (ngraph/flex/__init__.py:1-4,
call sites in ngraph/transformers/flexgputransform.py:78-157,347-371).

A flex16 tensor is int16 mantissas plus one shared exponent `dec`: value = mantissa * 2**-dec.
Rules (each reproduces the reference's flex golden tests):
  * dec is kept in [0, 31]; an unused tensor has dec 8; `fixed_point=True` pins dec 8 for good.
  * first write: the largest dec that holds the true (unsaturated) maximum of what is written;
    a zero maximum leaves dec 8.
  * after a write that saturated (max |mantissa| >= 32767): the next write uses dec - 2, and the
    history records twice the saturated value.
  * otherwise the next write uses the largest dec that holds
    max(history) + 3 * std(history) over the last 16 recorded maxima.
"""
import math
from collections import deque

STORAGE_BITS = 16
MANT_MAX = 2 ** 15 - 1
MANT_MIN = -2 ** 15
DEC_MIN, DEC_MAX = 0, 31
DEFAULT_DEC = 8
HISTORY_LEN = 16
HEADROOM_SIGMAS = 3.0


class Flex(object):
    """dtype descriptor (ngraph/flex/base.py:7-44)."""

    def __init__(self, storage_bits=STORAGE_BITS, exp_bits=5):
        self.storage_bits = storage_bits
        self.itemsize = storage_bits // 8
        self.type = "flex"
        self.str = "<i2"
        self.name = "flex"
        self.dtype_name = "flex"
        self.exp_bits = exp_bits
        self.pclip = 2 ** (storage_bits - 1) - 1
        self.nclip = -2 ** (storage_bits - 1)

    def __eq__(self, other):
        return isinstance(other, Flex) and self.storage_bits == other.storage_bits

    def __hash__(self):
        return hash(("flex", self.storage_bits))

    @staticmethod
    def get_scale(maxabs):
        d = largest_dec_holding(maxabs)
        return 2.0 ** -(DEFAULT_DEC if d is None else d)


flex16 = Flex()


def largest_dec_holding(maxabs):
    """Largest dec in [0, 31] with maxabs * 2**dec <= 32767; None when maxabs is 0."""
    a = float(maxabs)
    if a != a:
        return None
    if math.isinf(a):
        return DEC_MIN
    if a <= 0.0:
        return None
    # a = m * 2**e with 0.5 <= m < 1  ->  a * 2**dec <= 32767  <=>  dec <= 15 - e (+1 if it fits)
    m, e = math.frexp(a)
    dec = 15 - e
    if a * 2.0 ** (dec + 1) <= MANT_MAX:
        dec += 1
    while a * 2.0 ** dec > MANT_MAX:
        dec -= 1
    return DEC_MIN if dec < DEC_MIN else DEC_MAX if dec > DEC_MAX else dec


class FlexEntry(object):
    """Exponent state of one device buffer; all views of the buffer share it
    (ngraph/transformers/flexgputransform.py:211-221)."""

    def __init__(self, flex_id, name="", fixed_point=False):
        self.flex_id = flex_id
        self.name = name
        self.dtype = flex16
        self.fixed_point = fixed_point
        self.reset_entry()

    def reset_entry(self):
        self.dec = DEFAULT_DEC
        self.initialized = self.fixed_point
        self.pending_dec = None
        self.history = deque(maxlen=HISTORY_LEN)
        self.overflows = 0
        self._run_value = None      # last recorded maximum and how many times in a row it came
        self._run_length = 0

    @property
    def scale(self):
        return 2.0 ** -self.dec

    def dec_for_next_write(self):
        return self.dec if self.pending_dec is None else self.pending_dec

    def begin_write(self):
        """manage_before_computation: adopt the exponent chosen after the previous write."""
        if self.pending_dec is not None:
            self.dec = self.pending_dec
            self.pending_dec = None
        return self.dec

    def initialize_from_range(self, maxabs_real, from_host=False):
        """First write: exponent from the true range of the values about to be stored.  An
        all-zero HOST write (the initial value of a freshly created optimizer state) says nothing
        about the range: the default exponent is kept and the first write by a kernel measures
        again."""
        d = None if self.fixed_point else largest_dec_holding(maxabs_real)
        if d is not None:
            self.dec = d
        self.initialized = self.fixed_point or d is not None or not from_host
        return self.dec

    def end_write(self, maxabs_mantissa):
        """manage_after_computation: record this write's max |mantissa|, choose the next dec."""
        if self.fixed_point:
            return
        if maxabs_mantissa >= MANT_MAX:
            self.overflows += 1
            self._run_length = 0
            self.history.append(2.0 * maxabs_mantissa * self.scale)
            self.pending_dec = DEC_MIN if self.dec - 2 < DEC_MIN else self.dec - 2
            return
        value = maxabs_mantissa * self.scale
        if value == self._run_value:
            self._run_length += 1
            if self._run_length > HISTORY_LEN:
                # the window already holds nothing but this value: same mean, zero spread, same
                # choice as after the previous write (steady state of an inference loop)
                self.pending_dec = self._run_choice
                return
        else:
            self._run_value, self._run_length = value, 1
        self.history.append(value)
        hist = list(self.history)
        n = len(hist)
        mean = math.fsum(hist) / n
        var = math.fsum([(h - mean) ** 2 for h in hist]) / n
        predicted = builtin_max(hist) + HEADROOM_SIGMAS * math.sqrt(var)
        self.pending_dec = self._run_choice = largest_dec_holding(predicted)


builtin_max = max


class FlexManager(object):
    """Creates entries and hands out rows of the device scale table / statistics array."""

    default_dec = DEFAULT_DEC

    @staticmethod
    def fixed_point_resolution():
        return 2.0 ** -DEFAULT_DEC

    def __init__(self, fixed_point=False, verbose=False):
        self.fixed_point = fixed_point
        self.verbose = verbose
        self.flex_entries = {}
        self.autoflex_count = 0
        self.n_slots = 0

    def make_flex_entry(self, name=""):
        e = FlexEntry(len(self.flex_entries), name, self.fixed_point)
        self.flex_entries[e.flex_id] = e
        return e

    def new_slot(self):
        s = self.n_slots
        self.n_slots += 1
        return s
