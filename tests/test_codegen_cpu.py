"""No GPU needed: the C-ABI library loads, exports every declared symbol, and every kind of fused
program generates CUDA that NVRTC compiles for sm_100a."""
import itertools
import os
import re

import pytest

from ngraph_python_b200 import lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_header_symbols_exported():
    text = open(os.path.join(ROOT, "include", "b200ng.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set(re.findall(r"\b(b2_[a-z0-9_]+)\s*\(", text))
    assert len(names) >= 10
    raw = lib.raw()
    for n in sorted(names):
        assert hasattr(raw, n), "library does not export %s" % n
    assert lib.raw().b2_version() >= 100


def test_invalid_program_is_rejected():
    ins = [dict(dtype=lib.F32, strides=(0, 0, 1))]
    outs = [dict(dtype=lib.F32, strides=(0, 0, 1), reg=5)]   # undefined register
    prog = lib.make_program((1, 1, 64), ins, [], [("neg", 0, None)], outs, [], lib.REDUCE_NONE)
    with pytest.raises(lib.B200Error, match="undefined register"):
        lib.ew_check(prog)
    outs = [dict(dtype=lib.FLEX16, slot=-1, strides=(0, 0, 1), reg=1)]
    prog = lib.make_program((1, 1, 64), ins, [], [("neg", 0, None)], outs, [], lib.REDUCE_NONE)
    with pytest.raises(lib.B200Error, match="no slot"):
        lib.ew_check(prog)


MODES = [(lib.REDUCE_NONE, (3, 5, 64)), (lib.REDUCE_C, (1, 7, 4096)), (lib.REDUCE_C, (2, 9, 40)),
         (lib.REDUCE_C, (1, 1, 1 << 22)), (lib.REDUCE_B, (2, 33, 256))]


@pytest.mark.parametrize("mode_dims,flex,vec,probe",
                         list(itertools.product(MODES, (0, 1), (0, 1), (0, 1))))
def test_programs_compile(mode_dims, flex, vec, probe):
    mode, (A, B, Cn) = mode_dims
    dt = lib.FLEX16 if flex else lib.F32
    full = (B * Cn, Cn, 1)
    ins = [dict(dtype=dt, slot=0 if flex else -1, strides=full),
           dict(dtype=dt, slot=1 if flex else -1, strides=(0, 0, 1)),     # broadcast over A, B
           dict(dtype=lib.F32, strides=(B, 1, 0))]                        # broadcast over C
    ops = [("mul", 0, 1), ("add", 4, 2), ("tanh", 5, None), ("maximum", 6, 3), ("exp", 7, None)]
    outs = [dict(dtype=dt, slot=2 if flex else -1, strides=full, reg=8)]
    if mode == lib.REDUCE_NONE:
        reds = []
    elif mode == lib.REDUCE_C:
        st = (B, 1, 0)
        reds = [dict(dtype=dt, slot=3 if flex else -1, strides=st, reg=8, redop="sum"),
                dict(dtype=lib.F32, strides=st, reg=7, redop="argmax")]
    else:
        st = (Cn, 0, 1)
        reds = [dict(dtype=dt, slot=3 if flex else -1, strides=st, reg=8, redop="max"),
                dict(dtype=lib.F32, strides=st, reg=7, redop="argmin")]
    if mode == lib.REDUCE_C and Cn == 1 << 22:
        reds = reds[:1]   # the split variant has no arg reductions
    prog = lib.make_program((A, B, Cn), ins, [0.5], ops, outs, reds, mode)
    src = lib.ew_check(prog, vec=bool(vec), probe=bool(probe), want_source=True)
    assert "b2_ew_main" in src
    if mode == lib.REDUCE_C and Cn == 1 << 22:
        assert "b2_ew_finalize" in src
