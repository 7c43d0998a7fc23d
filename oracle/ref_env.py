"""Finds the reference tree and makes `import ngraph` work in this interpreter.

Test infrastructure (used by tests/, by the fixture generator and by the CPU-reference legs of
bench.py; never by the package).  Search order:
  1. the directory named by the environment variable B200NG_REFERENCE,
  2. oracle/_ref/ (made by oracle/make_ref.py from a checkout of NervanaSystems/ngraph-python).
`install()` goes through ngraph_python_b200.ngraph_compat (the unmodified reference was written
for Python 2.7/3.5 and numpy 1.x), which puts the tree on sys.path.
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def reference_root():
    """Directory that holds the reference's `ngraph` package, or None."""
    cands = [os.environ.get("B200NG_REFERENCE"), os.path.join(HERE, "_ref")]
    for c in cands:
        if c and os.path.isdir(os.path.join(c, "ngraph")):
            return os.path.abspath(c)
    return None


def install():
    """Returns the reference root after making it importable, or None when there is none."""
    root = reference_root()
    if root is None:
        return None
    repo = os.path.dirname(HERE)
    if repo not in sys.path:
        sys.path.insert(0, repo)
    from ngraph_python_b200 import ngraph_compat
    ngraph_compat.install(root)
    resnet_dir = os.path.join(root, "examples", "resnet")
    if os.path.isdir(resnet_dir) and resnet_dir not in sys.path:
        sys.path.insert(0, resnet_dir)
    return root
