"""Lets an unmodified nGraph-Python tree (v0.4.0, written for Python 2.7/3.5 and numpy 1.x) import
on a current interpreter, so that the `b200` plug-in (ngraph_plugin.py) can be used with it.

    from ngraph_python_b200 import ngraph_compat
    ngraph_compat.install("/path/to/ngraph-python")     # or install() if ngraph is on sys.path
    import ngraph

What it does, all at import level and none of it touching the reference's files:
  * restores the names the reference still takes from `collections`, `numpy` and `inspect`
    (ngraph/transformers/base.py:128-130 uses collections.Sequence, for instance);
  * selects the pure-Python protobuf implementation (the checked-in *_pb2.py files predate the
    C++ one's checks);
  * appends this directory to sys.path, where small stand-ins live for third-party packages the
    reference imports (future.utils, orderedset, cached_property, frozendict, monotonic, appdirs,
    configargparse, parsel, h5py).  They are found only when the real package is not installed.
"""
import collections
import collections.abc
import inspect
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def install(reference_root=None):
    """reference_root: directory holding the `ngraph` package, put in front of sys.path; None
    when `ngraph` is importable already."""
    os.environ.setdefault("PROTOCOL_BUFFERS_PYTHON_IMPLEMENTATION", "python")
    for name in ("Iterable", "Sequence", "Set", "Mapping", "MutableMapping", "MutableSet",
                 "MutableSequence", "Callable", "Hashable", "Sized", "Container", "Iterator"):
        if not hasattr(collections, name):
            setattr(collections, name, getattr(collections.abc, name))
    import numpy as np
    for alias, target in (("float", float), ("int", int), ("bool", bool), ("object", object),
                          ("str", str)):
        if alias not in np.__dict__:
            setattr(np, alias, target)
    if not hasattr(inspect, "getargspec"):
        inspect.getargspec = inspect.getfullargspec
    if reference_root is not None and reference_root not in sys.path:
        sys.path.insert(0, reference_root)
    if HERE not in sys.path:
        sys.path.append(HERE)
