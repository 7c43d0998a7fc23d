"""Hashable immutable mapping for the reference's imports."""
from collections.abc import Mapping


class frozendict(Mapping):
    def __init__(self, *a, **kw):
        self._d = dict(*a, **kw)
        self._h = None

    def __getitem__(self, k):
        return self._d[k]

    def __iter__(self):
        return iter(self._d)

    def __len__(self):
        return len(self._d)

    def __hash__(self):
        if self._h is None:
            self._h = hash(frozenset(self._d.items()))
        return self._h

    def copy(self, **add):
        return frozendict(self._d, **add)

    def __repr__(self):
        return "frozendict(%r)" % (self._d,)
