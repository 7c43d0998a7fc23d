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

Not collected by this repository's own test run; tests/test_reference_suites_gpu.py runs it in a
child process and holds the outcome to what the reference's own cpu transformer passes.
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


class _LegacyParam(object):
    """A parameter value with a mark on it, written the way pytest 3 allowed --
    `pytest.config.flex_disabled(value)` inside a parametrize list -- until the number of argument
    names is known (one name: the value is the parameter; several: it is the tuple of them)."""

    def __init__(self, value, mark):
        self.value, self.mark = value, mark

    def to_param(self, n_names):
        if n_names == 1:
            return pytest.param(self.value, marks=self.mark)
        return pytest.param(*self.value, marks=self.mark)


class _LegacyMark(object):
    """The mark objects the reference's conftest hangs on `pytest.config` (flex_disabled,
    argon_disabled, ...), usable in all the ways its tests use them: as a decorator, called with
    keywords (`reason=`) to refine it, and called with a parameter value to mark that value."""

    def __init__(self, decorator):
        self.decorator = decorator

    @property
    def mark(self):
        """What pytest reads when the object stands in a `pytestmark` list."""
        return self.decorator.mark

    def __call__(self, *args, **kwargs):
        if len(args) == 1 and not kwargs and (isinstance(args[0], type) or
                                              type(args[0]).__name__ == "function"):
            return self.decorator(args[0])
        if args:
            deco = self.decorator.with_args(**kwargs) if kwargs else self.decorator
            return _LegacyParam(args[-1], deco)
        return _LegacyMark(self.decorator.with_args(**kwargs))

    def __getattr__(self, name):
        return getattr(self.decorator, name)


def _legacy_parametrize():
    from _pytest.python import Metafunc
    if getattr(Metafunc.parametrize, "_b200ng_legacy", False):
        return
    plain = Metafunc.parametrize

    def parametrize(self, argnames, argvalues, *args, **kwargs):
        names = [n.strip() for n in argnames.split(",") if n.strip()] \
            if isinstance(argnames, str) else list(argnames)
        argvalues = [v.to_param(len(names)) if isinstance(v, _LegacyParam) else v
                     for v in argvalues]
        return plain(self, argnames, argvalues, *args, **kwargs)
    parametrize._b200ng_legacy = True
    Metafunc.parametrize = parametrize


def _python3_helpers():
    """ngraph/testing/flex_util.py:73-98 names test cases after `function.func_name`, which
    Python 3 spells `__name__`."""
    from types import FunctionType
    import ngraph.testing.flex_util as flex_util
    plain = flex_util.id_func
    if getattr(plain, "_b200ng_py3", False):
        return

    def id_func(param):
        if isinstance(param, FunctionType):
            return param.__name__.title()
        return plain(param)
    id_func._b200ng_py3 = True
    flex_util.id_func = id_func


FLEX_TRANSFORMERS = ("flexgpu", "b200flex")


@pytest.hookimpl(tryfirst=True)
def pytest_configure(config):
    pytest.config = config           # what `pytest.config.getoption(...)` in the reference reads
    _python3_helpers()


def pytest_sessionstart(session):
    config = session.config
    # after the reference's conftest has made its marks (conftest.py:85-106): the same marks,
    # usable under today's pytest, and counting this package's flex transformer as a flex one.
    # Its known-failure marks are strict for its own transformer only: a case that works here
    # shows up as xpassed instead of failing the run.
    name = config.getvalue("transformer")
    flex, argon = name in FLEX_TRANSFORMERS, name == "argon"
    strict = name in ("flexgpu", "argon")
    x = pytest.mark.xfail
    config.flex_and_argon_disabled = _LegacyMark(
        x(flex or argon, reason="Not supported by argon or flex backend", strict=strict))
    config.argon_disabled = _LegacyMark(
        x(argon, reason="Not supported by argon backend", strict=strict))
    config.flex_disabled = _LegacyMark(x(flex, reason="Failing test for Flex", strict=strict))
    config.hetr_and_cpu_enabled_only = _LegacyMark(
        x(name not in ("hetr", "cpu"), reason="Only Hetr/CPU and CPU transformers supported",
          strict=True))
    config.flex_skip = _LegacyMark(pytest.mark.skipif(flex, reason="Randomly failing test for Flex"))
    config.argon_skip = _LegacyMark(pytest.mark.skipif(argon, reason="argon"))
    config.flex_skip_now = pytest.skip if flex else (lambda *a, **k: None)
    _legacy_parametrize()


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
