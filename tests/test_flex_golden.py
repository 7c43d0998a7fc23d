"""The CPU flex oracle against every golden vector of the reference's flex elementwise tests."""
import numpy as np
import pytest

from tests.flexsim import FlexSimExecutor, flex_tolerance
from tests.golden.flex_vectors import CASES, STATE_FACTS


def _id(case):
    op, calls, src = case
    return "%s@%s" % (op, src.split("/")[-1])


@pytest.mark.parametrize("case", CASES, ids=_id)
def test_golden_case(case):
    op, calls, src = case
    ex = FlexSimExecutor(op, len(calls[0][0]))
    iterations = len(calls) != 1
    for operands, expected in calls:
        got = ex(*operands)
        if iterations:
            atol, rtol = flex_tolerance(expected)
            np.testing.assert_allclose(got, np.asarray(expected, dtype=np.float64),
                                       rtol=rtol, atol=atol, err_msg="%s %s" % (src, operands))
        else:
            assert np.array_equal(got, np.asarray(expected, dtype=np.float64)), \
                "%s %s: got %r expected %r" % (src, operands, got, expected)


def _first_multicall(op):
    if op == "sub_short":
        return [c for c in CASES if c[0] == "sub" and len(c[1]) == 4][0]
    return [c for c in CASES if c[0] == op and len(c[1]) > 1][0]


@pytest.mark.parametrize("fact", STATE_FACTS, ids=lambda f: "%s-%d-%s" % f[:3])
def test_state_fact(fact):
    op, idx, what, expected = fact
    case = _first_multicall(op)
    real_op = case[0]
    ex = FlexSimExecutor(real_op, len(case[1][0][0]))
    for i, (operands, _) in enumerate(case[1]):
        got = ex(*operands)
        if i == idx:
            if what == "result":
                assert float(got) == expected
            else:
                k = int(what[-1])
                assert float(ex.ph[k].host_read()) == expected
            return
    raise AssertionError("call index out of range")
