"""The exponent manager's two paths -- one entry at a time (FlexEntry.begin_write / end_write) and
many entries at once (FlexManager.begin_write_batch / end_write_batch, what a computation with
hundreds of written tensors uses) -- make the same choices, and both follow the oracle's manager
(oracle/flex_oracle.py: the rule that reproduces the reference's flex golden vectors)."""
import numpy as np

from ngraph_python_b200 import flex as F
from oracle import flex_oracle as fx


def _sequences(rng, n_entries, n_steps):
    """Per entry a series of true maxima |value| of what a kernel writes: drifting magnitudes,
    runs of one repeated value (an inference loop), jumps that saturate, zeros, values that sit
    on a power of two."""
    out = np.zeros((n_steps, n_entries))
    for j in range(n_entries):
        kind = j % 5
        level = rng.uniform(0.01, 100.0)
        for s in range(n_steps):
            if kind == 0:
                level *= rng.uniform(0.7, 1.4)
                out[s, j] = level
            elif kind == 1:
                out[s, j] = 3.21 if s % 40 < 30 else rng.uniform(0.1, 10.0)
            elif kind == 2:
                out[s, j] = level * (16.0 if rng.rand() < 0.2 else rng.uniform(0.5, 1.0))
            elif kind == 3:
                out[s, j] = 0.0 if s < 3 else rng.uniform(0.5, 0.6)
            else:
                out[s, j] = 2.0 if s % 2 else 2.0 - 2.0 ** -12
    return out


def _mantissas(real, dec):
    """max |mantissa| a kernel reports for true maxima `real` stored with exponents `dec`."""
    return np.minimum(np.rint(real * 2.0 ** dec.astype(np.float64)), 32768).astype(np.int64)


def test_batch_path_makes_the_choices_of_the_one_entry_path():
    rng = np.random.RandomState(0)
    n, steps = 300, 120
    seq = _sequences(rng, n, steps)
    one, many = F.FlexManager(), F.FlexManager()
    e1 = [one.make_flex_entry("t%d" % i) for i in range(n)]
    for _ in range(n):
        many.make_flex_entry()
    ids = np.arange(n, dtype=np.int64)
    for m in (one, many):
        m.initialized[:n] = True
    long_runs = False
    for s in range(steps):
        d1 = np.array([e.begin_write() for e in e1])
        d2 = many.begin_write_batch(ids)
        assert np.array_equal(d1, d2), "step %d: exponents used differ" % s
        mant = _mantissas(seq[s], d1)
        for e, v in zip(e1, mant):
            e.end_write(int(v))
        many.end_write_batch(ids, mant)
        assert np.array_equal(one.pending[:n], many.pending[:n]), "step %d" % s
        assert np.array_equal(one.run_length[:n], many.run_length[:n])
        assert np.array_equal(one.overflows[:n], many.overflows[:n])
        assert one.settled(ids) == many.settled(ids)
        long_runs = long_runs or bool((many.run_length[:n] > F.HISTORY_LEN).any())
    assert many.overflows[:n].sum() > 0 and long_runs          # the sequences reached both rules


def test_batch_path_on_a_subset_leaves_the_other_entries_alone():
    m = F.FlexManager()
    for _ in range(70):                          # more than the first allocation: arrays grow
        m.make_flex_entry()
    ids = np.array([3, 64, 69], dtype=np.int64)
    m.initialized[ids] = True
    m.end_write_batch(ids, np.array([100, 32767, 20000]))
    assert list(m.hist_len[ids]) == [1, 1, 1] and m.hist_len.sum() == 3
    assert m.pending[64] == F.DEFAULT_DEC - 2 and m.pending[0] == -1
    assert m.flex_entries[69].history == [20000 * 2.0 ** -8]


def test_one_entry_path_follows_the_oracle_manager():
    rng = np.random.RandomState(1)
    seq = _sequences(rng, 40, 80)
    for j in range(seq.shape[1]):
        mine, ref = F.FlexEntry(j), fx.FlexEntry()
        first = float(rng.uniform(0.01, 500.0))
        mine.initialize_from_range(first)
        ref.initialize(first)
        assert mine.dec == ref.dec
        for s in range(seq.shape[0]):
            mine.begin_write()
            ref.prepare_write()
            assert mine.dec == ref.dec, "entry %d step %d" % (j, s)
            mant = int(_mantissas(seq[s, j:j + 1], np.array([mine.dec]))[0])
            mine.end_write(mant)
            ref.observe(mant)


def _bookkeeping_transformer(ng, builder, **kw):
    """A planned (not executable) flex16 computation whose exponent bookkeeping can run on the
    host: scale table and statistics as CPU tensors."""
    import torch
    outs, params, _ = builder(ng, **kw)
    t = ng.transformers.allocate_transformer("b200", flex=True, plan_only=True)
    comp = t.computation(outs, *params)
    t.initialize()
    n = t.flex_manager.n_slots + 8
    t._table = torch.zeros((n, 2), dtype=torch.float32)
    t._stats = torch.zeros((n,), dtype=torch.int32)
    t._table_host = torch.zeros((n, 2), dtype=torch.float32)
    t._stats_host = torch.zeros((n,), dtype=torch.int32)
    t._table_np = t._table_host.numpy()
    t._dec_uploaded = np.full((n,), -1, dtype=np.int64)
    t._table_dirty = True
    for b in t._buffers.values():
        if b.entry is not None:
            b.entry.initialized = True
    return t, comp


def test_call_bookkeeping_follows_the_rule_entry_by_entry():
    """The transformer's per-call bookkeeping (array operations over all written tensors) against
    the plain restatement: before a call every written tensor adopts its pending exponent and its
    table rows follow; after it every written tensor records its maximum."""
    import ngraph_python_b200 as ng
    from tests.golden import cases
    t, comp = _bookkeeping_transformer(ng, cases.resnet8_small)
    written = [b for b in comp.written]
    assert len(written) > 15
    # the restatement keeps its own entries, fed with the same statistics
    mirror = {id(b): F.FlexEntry(k) for k, b in enumerate(written)}
    for m in mirror.values():
        m.initialized = True
    rng = np.random.RandomState(5)
    level = {id(b): rng.uniform(0.05, 50.0) for b in written}
    steady_seen = False
    for call in range(60):
        t._begin_call_flex(comp)
        for b in written:
            want = mirror[id(b)].begin_write()
            assert b.entry.dec == want, "call %d, %s" % (call, b.name)
            assert t._table_np[b.slot_write, 0] == 2.0 ** -want
            assert t._table_np[b.slot_write, 1] == 2.0 ** want
        assert not t._table_dirty                 # uploaded (to the CPU stand-in of the table)
        assert np.array_equal(t._table.numpy(), t._table_np)
        stats = t._stats_host.numpy()
        for b in written:
            if call < 25:
                level[id(b)] *= rng.uniform(0.8, 1.3)        # a drifting range, then a fixed one
            m = int(min(np.rint(level[id(b)] * 2.0 ** b.entry.dec), 32768))
            stats[b.slot_write] = m
            mirror[id(b)].end_write(m)
        t._end_call_flex(comp)
        for b in written:
            assert b.entry.pending_dec == mirror[id(b)].pending_dec, "call %d, %s" % (call, b.name)
        steady_seen = steady_seen or comp._steady is not None
    assert steady_seen                            # a fixed range ends in the steady-state path
    t.close()
