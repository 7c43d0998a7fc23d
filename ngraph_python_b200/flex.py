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


def _choose_dec_scalar(hist):
    """The rule for a write that did not saturate, on a list of recorded maxima: largest dec that
    holds max + 3 standard deviations (exactly summed)."""
    n = len(hist)
    mean = math.fsum(hist) / n
    var = math.fsum([(h - mean) ** 2 for h in hist]) / n
    return largest_dec_holding(builtin_max(hist) + HEADROOM_SIGMAS * math.sqrt(var))


builtin_max = max
_NONE = -1          # "no exponent chosen" in the integer arrays below


class FlexManager(object):
    """Creates entries, hands out rows of the device scale table / statistics array, and holds
    the exponent state of ALL entries in arrays, so that the bookkeeping of a computation with
    hundreds of written tensors (a training step) is a handful of numpy operations per call
    (`begin_write_batch`, `end_write_batch`) instead of a Python loop over entries -- that loop
    took 1.2 ms per ResNet-20 training step, with the GPU idle.  A FlexEntry is a view on one
    row of these arrays; its own methods apply the same rules one entry at a time (first writes,
    host writes, tests) and the two paths make the same choices."""

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
        self._alloc(64)

    def _alloc(self, cap):
        import numpy as np
        old = getattr(self, "dec", None)
        n = 0 if old is None else len(old)

        def grow(name, dtype, fill, shape=()):
            new = np.full((cap,) + shape, fill, dtype=dtype)
            if n:
                new[:n] = getattr(self, name)
            setattr(self, name, new)
        grow("dec", np.int64, DEFAULT_DEC)
        grow("pending", np.int64, _NONE)
        grow("initialized", np.bool_, False)
        grow("overflows", np.int64, 0)
        grow("hist", np.float64, 0.0, (HISTORY_LEN,))     # ring of the last recorded maxima
        grow("hist_len", np.int64, 0)
        grow("hist_pos", np.int64, 0)
        grow("run_value", np.float64, np.nan)              # nan: no value recorded yet
        grow("run_length", np.int64, 0)
        grow("run_choice", np.int64, _NONE)

    def make_flex_entry(self, name=""):
        i = len(self.flex_entries)
        if i >= len(self.dec):
            self._alloc(2 * len(self.dec))
        e = FlexEntry(i, name, self.fixed_point, manager=self)
        self.flex_entries[i] = e
        return e

    def new_slot(self):
        s = self.n_slots
        self.n_slots += 1
        return s

    # -- one row --------------------------------------------------------------------------------
    def _push(self, i, value):
        pos = self.hist_pos[i]
        self.hist[i, pos] = value
        self.hist_pos[i] = (pos + 1) % HISTORY_LEN
        if self.hist_len[i] < HISTORY_LEN:
            self.hist_len[i] += 1

    def history_of(self, i):
        """The recorded maxima of entry i, oldest first."""
        n, pos = int(self.hist_len[i]), int(self.hist_pos[i])
        row = self.hist[i]
        if n < HISTORY_LEN:
            return [float(v) for v in row[:n]]
        return [float(v) for v in list(row[pos:]) + list(row[:pos])]

    # -- many rows at once ----------------------------------------------------------------------
    def begin_write_batch(self, ids):
        """FlexEntry.begin_write for the entries `ids` (int array, no duplicates): returns the
        exponents their next write uses."""
        p = self.pending[ids]
        has = p >= 0
        if has.any():
            sel = ids[has]
            self.dec[sel] = p[has]
            self.pending[sel] = _NONE
        return self.dec[ids]

    def end_write_batch(self, ids, maxima):
        """FlexEntry.end_write for the entries `ids` (int array, no duplicates) with the max
        |mantissa| each of them recorded."""
        import numpy as np
        if self.fixed_point or len(ids) == 0:
            return
        ids = np.asarray(ids, dtype=np.int64)
        m = np.asarray(maxima, dtype=np.int64)
        dec = self.dec[ids]
        scale = np.ldexp(1.0, (-dec).astype(np.int32))
        value = m * scale
        ovf = m >= MANT_MAX
        if ovf.any():
            sel = ids[ovf]
            self.overflows[sel] += 1
            self.run_length[sel] = 0
            self._push_many(sel, 2.0 * value[ovf])
            self.pending[sel] = np.maximum(dec[ovf] - 2, DEC_MIN)
        ok = ~ovf
        same = ok & (value == self.run_value[ids])
        if same.any():
            self.run_length[ids[same]] += 1
        # the window already holds nothing but this value: same choice as after the previous write
        early = same & (self.run_length[ids] > HISTORY_LEN)
        if early.any():
            sel = ids[early]
            self.pending[sel] = self.run_choice[sel]
        fresh = ok & ~same
        if fresh.any():
            sel = ids[fresh]
            self.run_value[sel] = value[fresh]
            self.run_length[sel] = 1
        rest = ok & ~early
        if not rest.any():
            return
        sel = ids[rest]
        self._push_many(sel, value[rest])
        H = self.hist[sel]
        n = self.hist_len[sel]
        mask = np.arange(HISTORY_LEN)[None, :] < n[:, None]     # rows fill from slot 0
        mean = H.sum(axis=1) / n                                 # unused slots hold 0
        d = np.where(mask, H - mean[:, None], 0.0)
        var = (d * d).sum(axis=1) / n
        predicted = np.where(mask, H, -np.inf).max(axis=1) + HEADROOM_SIGMAS * np.sqrt(var)
        choice = _largest_dec_holding_many(predicted)
        # numpy's sums are not the exactly rounded ones of the one-entry rule: where the value
        # lies within a hair of the point at which the choice changes, decide with that rule
        with np.errstate(over="ignore", invalid="ignore"):
            c = np.where(choice < 0, 0, choice).astype(np.int32)
            t0 = np.ldexp(predicted, c)
            t1 = np.ldexp(predicted, c + 1)
        near = (choice >= 0) & ((np.abs(t0 - MANT_MAX) < 1e-6 * MANT_MAX) |
                                (np.abs(t1 - MANT_MAX) < 1e-6 * MANT_MAX))
        for k in np.nonzero(near)[0]:
            exact = _choose_dec_scalar(self.history_of(int(sel[k])))
            choice[k] = _NONE if exact is None else exact
        self.pending[sel] = choice
        self.run_choice[sel] = choice

    def _push_many(self, sel, values):
        pos = self.hist_pos[sel]
        self.hist[sel, pos] = values
        self.hist_pos[sel] = (pos + 1) % HISTORY_LEN
        self.hist_len[sel] = builtin_min_arr(self.hist_len[sel] + 1)

    def settled(self, ids):
        """True when every one of the entries has seen the same maximum for longer than the
        history window and will keep its exponent: nothing can change while that lasts."""
        if self.fixed_point:
            return True
        p, d = self.pending[ids], self.dec[ids]
        return bool(((self.run_length[ids] > HISTORY_LEN) & ((p < 0) | (p == d))).all())


def builtin_min_arr(a):
    import numpy as np
    return np.minimum(a, HISTORY_LEN)


def _largest_dec_holding_many(a):
    """largest_dec_holding over an array of non-negative finite values; -1 where it gives None."""
    import numpy as np
    a = np.asarray(a, dtype=np.float64)
    out = np.full(a.shape, _NONE, dtype=np.int64)
    pos = a > 0.0
    if not pos.any():
        return out
    x = a[pos]
    _, e = np.frexp(x)
    dec = 15 - e.astype(np.int64)
    with np.errstate(over="ignore"):
        up = np.ldexp(x, (dec + 1).astype(np.int32)) <= MANT_MAX
        dec = np.where(up, dec + 1, dec)
        for _ in range(2):
            down = np.ldexp(x, dec.astype(np.int32)) > MANT_MAX
            dec = np.where(down, dec - 1, dec)
    dec = np.clip(dec, DEC_MIN, DEC_MAX)
    dec = np.where(np.isinf(x), DEC_MIN, dec)
    out[pos] = dec
    return out


class FlexEntry(object):
    """Exponent state of one device buffer; all views of the buffer share it
    (ngraph/transformers/flexgputransform.py:211-221).  The state lives in row `flex_id` of the
    manager's arrays."""

    def __init__(self, flex_id, name="", fixed_point=False, manager=None):
        if manager is None:                       # a stand-alone entry: a manager of its own
            manager = FlexManager(fixed_point=fixed_point)
            manager.flex_entries[0] = self
            flex_id_row = 0
        else:
            flex_id_row = flex_id
        self.m = manager
        self.i = flex_id_row
        self.flex_id = flex_id
        self.name = name
        self.dtype = flex16
        self.fixed_point = fixed_point
        self.reset_entry()

    def reset_entry(self):
        m, i = self.m, self.i
        m.dec[i] = DEFAULT_DEC
        m.initialized[i] = self.fixed_point
        m.pending[i] = _NONE
        m.hist[i] = 0.0
        m.hist_len[i] = 0
        m.hist_pos[i] = 0
        m.overflows[i] = 0
        m.run_value[i] = float("nan")
        m.run_length[i] = 0
        m.run_choice[i] = _NONE

    # -- state, as attributes ---------------------------------------------------------------------
    @property
    def dec(self):
        return int(self.m.dec[self.i])

    @dec.setter
    def dec(self, v):
        self.m.dec[self.i] = v

    @property
    def pending_dec(self):
        p = int(self.m.pending[self.i])
        return None if p < 0 else p

    @pending_dec.setter
    def pending_dec(self, v):
        self.m.pending[self.i] = _NONE if v is None else v

    @property
    def initialized(self):
        return bool(self.m.initialized[self.i])

    @initialized.setter
    def initialized(self, v):
        self.m.initialized[self.i] = bool(v)

    @property
    def overflows(self):
        return int(self.m.overflows[self.i])

    @property
    def history(self):
        return self.m.history_of(self.i)

    @property
    def _run_length(self):
        return int(self.m.run_length[self.i])

    @property
    def scale(self):
        return 2.0 ** -self.dec

    def dec_for_next_write(self):
        p = self.pending_dec
        return self.dec if p is None else p

    def begin_write(self):
        """manage_before_computation: adopt the exponent chosen after the previous write."""
        p = self.pending_dec
        if p is not None:
            self.dec = p
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
        m, i = self.m, self.i
        if maxabs_mantissa >= MANT_MAX:
            m.overflows[i] += 1
            m.run_length[i] = 0
            m._push(i, 2.0 * maxabs_mantissa * self.scale)
            self.pending_dec = DEC_MIN if self.dec - 2 < DEC_MIN else self.dec - 2
            return
        value = maxabs_mantissa * self.scale
        if value == m.run_value[i]:
            m.run_length[i] += 1
            if m.run_length[i] > HISTORY_LEN:
                # the window already holds nothing but this value: same mean, zero spread, same
                # choice as after the previous write (steady state of an inference loop)
                m.pending[i] = m.run_choice[i]
                return
        else:
            m.run_value[i] = value
            m.run_length[i] = 1
        m._push(i, value)
        choice = _choose_dec_scalar(m.history_of(i))
        choice = _NONE if choice is None else choice
        m.pending[i] = choice
        m.run_choice[i] = choice
