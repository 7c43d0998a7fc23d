"""Minimal ordered set (insertion ordered, indexable) for the reference's imports."""
from collections.abc import MutableSet, Sequence


class OrderedSet(MutableSet, Sequence):
    def __init__(self, iterable=None):
        self._d = {}
        if iterable is not None:
            self.update(iterable)

    def __len__(self):
        return len(self._d)

    def __contains__(self, x):
        return x in self._d

    def __iter__(self):
        return iter(self._d)

    def __reversed__(self):
        return reversed(list(self._d))

    def __getitem__(self, i):
        items = list(self._d)
        if isinstance(i, slice):
            return OrderedSet(items[i])
        return items[i]

    def add(self, x):
        self._d[x] = None

    def update(self, *iterables):
        for it in iterables:
            for x in it:
                self._d[x] = None

    def discard(self, x):
        self._d.pop(x, None)

    def remove(self, x):
        del self._d[x]

    def pop(self, last=True):
        if not self._d:
            raise KeyError("pop from an empty set")
        key = next(reversed(self._d)) if last else next(iter(self._d))
        del self._d[key]
        return key

    def index(self, x):
        return list(self._d).index(x)

    def copy(self):
        return OrderedSet(self._d)

    def clear(self):
        self._d.clear()

    def union(self, *others):
        r = self.copy()
        r.update(*others)
        return r

    def intersection(self, *others):
        r = OrderedSet()
        for x in self:
            if all(x in o for o in others):
                r.add(x)
        return r

    def difference(self, *others):
        r = OrderedSet()
        for x in self:
            if not any(x in o for o in others):
                r.add(x)
        return r

    def issubset(self, other):
        return all(x in other for x in self)

    def issuperset(self, other):
        return all(x in self for x in other)

    def __eq__(self, other):
        if isinstance(other, OrderedSet):
            return list(self) == list(other)
        try:
            return set(self) == set(other)
        except TypeError:
            return False

    def __ne__(self, other):
        return not self == other

    __hash__ = None

    def __repr__(self):
        return "OrderedSet(%r)" % (list(self._d),)
