from time import monotonic  # noqa: F401
