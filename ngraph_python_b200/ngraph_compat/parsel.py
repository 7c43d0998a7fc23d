class Selector(object):
    def __init__(self, *a, **kw):
        raise NotImplementedError("parsel stub")
