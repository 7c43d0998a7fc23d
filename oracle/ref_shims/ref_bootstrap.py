"""Import-time compatibility layer that lets the unmodified nGraph-Python tree (v0.4.0, written
for Python 2.7/3.5 and numpy 1.x) import on Python 3.12 + numpy 2.  Used only by the scripts
that generate golden fixtures; nothing in the product imports it.

Usage:  import ref_bootstrap; ref_bootstrap.install(reference_root)
"""
import collections
import collections.abc
import inspect
import os
import sys


def install(reference_root):
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
    here = os.path.dirname(os.path.abspath(__file__))
    for p in (reference_root, here):
        if p not in sys.path:
            sys.path.insert(0, p)
