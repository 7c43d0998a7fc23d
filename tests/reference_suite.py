"""Runs the reference's own transformer-dependent tests against a transformer of choice.

    python tests/reference_suite.py --transformer b200 [--report FILE] [--marker EXPR]
                                    [directories of the reference tree] [-k expr] [pytest args]

The tests are the reference's, untouched (tests/transformer_dependent, frontends/neon/tests and
frontends/common/tests of the tree that oracle/ref_env.py finds); the marker expression is the one its
Makefile uses for the GPU transformer (Makefile:173-189: "transformer_dependent and not flex_only
and not hetr_only").  The reference's conftest.py and test modules were written for a pytest that
exposed the active configuration as `pytest.config`; this module is loaded as a plug-in before
them and puts that attribute back.  It also imports the b200 plug-in first, so that 'b200' is
among the `--transformer` choices the reference's conftest offers.

Not collected by this repository's own test run: the outcome of the reference's suite on b200 is
recorded in DESIGN.md, test by test where it fails.
"""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import pytest  # noqa: E402

from oracle import ref_env  # noqa: E402

REF = ref_env.install()
if REF is not None:
    import ngraph_python_b200.ngraph_plugin  # noqa: E402,F401


@pytest.hookimpl(tryfirst=True)
def pytest_configure(config):
    pytest.config = config           # what `pytest.config.getoption(...)` in the reference reads


_outcomes = {}


def pytest_runtest_logreport(report):
    """One line per test for --report: the worst of its set-up / call / tear-down outcomes."""
    rank = {"passed": 0, "skipped": 1, "failed": 2}
    if getattr(report, "wasxfail", None) is not None and report.outcome != "failed":
        outcome = "xfailed"
    else:
        outcome = "error" if (report.outcome == "failed" and report.when != "call") else \
            report.outcome
    prev = _outcomes.get(report.nodeid)
    order = {"passed": 0, "xfailed": 1, "skipped": 1, "failed": 2, "error": 3}
    if prev is None or order.get(outcome, 0) > order.get(prev, 0):
        _outcomes[report.nodeid] = outcome
    del rank


def main(argv):
    if REF is None:
        sys.exit("no reference tree: run oracle/make_ref.py first")
    transformer, report, marker_arg = "b200", None, None
    rest = []
    it = iter(argv)
    for a in it:
        if a == "--transformer":
            transformer = next(it)
        elif a == "--report":
            report = os.path.abspath(next(it))
        elif a == "--marker":
            marker_arg = next(it)
        else:
            rest.append(a)
    targets = [a for a in rest if not a.startswith("-") and os.path.exists(os.path.join(REF, a))]
    rest = [a for a in rest if a not in targets]
    if not targets:
        targets = [os.path.join("tests", "transformer_dependent")]
    marker = "transformer_dependent and not flex_only and not hetr_only and not hetr_gpu_only"
    if marker_arg is not None:          # e.g. --marker "not hetr_only and not flex_only"
        marker = marker_arg
    args = ["-p", "tests.reference_suite", "--rootdir", REF, "-c", os.path.join(REF, "pytest.ini"),
            "--transformer", transformer, "-m", marker, "-q", "-W", "ignore",
            "-o", "cache_dir=/tmp/b200ng_ref_suite_cache"] + rest + \
           [os.path.join(REF, t) for t in targets]
    os.chdir(REF)
    rc = pytest.main(args)
    if report:
        mod = sys.modules.get("tests.reference_suite")
        outcomes = getattr(mod, "_outcomes", _outcomes)
        with open(report, "w") as f:
            for nodeid in sorted(outcomes):
                f.write("%s %s\n" % (outcomes[nodeid], nodeid))
    return rc


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
