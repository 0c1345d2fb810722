"""``galvatron.core`` under its reference name (galvatron/core/__init__.py:1-17): the profilers, the runtime API,
the search engine and the argument entry points, all provided by ``hetu_galvatron_b200.core``."""
import importlib

_core = importlib.import_module("hetu_galvatron_b200.core")

__all__ = list(_core.__all__)


def __getattr__(name):
    return getattr(_core, name)


def __dir__():
    return sorted(set(globals()) | set(__all__))
