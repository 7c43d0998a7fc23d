"""Minimal stand-in for the `future.utils` names the reference imports."""
PY2 = False
PY3 = True
native_str = str


def with_metaclass(meta, *bases):
    class metaclass(meta):
        def __new__(cls, name, this_bases, d):
            return meta(name, bases, d)
    return type.__new__(metaclass, "temporary_class", (), {})


def iteritems(d, **kw):
    return iter(d.items(**kw))


def itervalues(d, **kw):
    return iter(d.values(**kw))


def iterkeys(d, **kw):
    return iter(d.keys(**kw))


def viewitems(d):
    return d.items()


def viewkeys(d):
    return d.keys()


def viewvalues(d):
    return d.values()
