"""argparse-backed stand-in for the configargparse names the reference imports."""
import argparse
from argparse import ArgumentDefaultsHelpFormatter  # noqa: F401

_DROP_INIT = ("default_config_files", "add_config_file_help", "ignore_unknown_config_file_keys",
              "config_file_parser_class", "args_for_setting_config_path", "auto_env_var_prefix")


class ArgumentParser(argparse.ArgumentParser):
    def __init__(self, *a, **kw):
        for k in _DROP_INIT:
            kw.pop(k, None)
        super().__init__(*a, **kw)

    def add_argument(self, *a, **kw):
        kw.pop("is_config_file", None)
        kw.pop("env_var", None)
        return super().add_argument(*a, **kw)

    def add_argument_group(self, *a, **kw):
        g = super().add_argument_group(*a, **kw)
        orig = g.add_argument

        def add_argument(*aa, **kk):
            kk.pop("is_config_file", None)
            kk.pop("env_var", None)
            return orig(*aa, **kk)
        g.add_argument = add_argument
        return g


ArgParser = ArgumentParser
