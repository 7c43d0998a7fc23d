import os


def user_cache_dir(appname=None, appauthor=None):
    return os.path.join(os.path.expanduser("~"), ".cache", appname or "app")
