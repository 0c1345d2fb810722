"""Import alias: lets programs written against the reference's package name run on this framework.

    import galvatron
    from galvatron.core import initialize_galvatron, GalvatronSearchEngine, construct_hybrid_parallel_model_api

Installed as a top-level package by ``pip install .``; from a checkout, add ``compat/`` to ``PYTHONPATH``.
Every name resolves to its counterpart in ``hetu_galvatron_b200`` (reference: galvatron/__init__.py,
galvatron/core/__init__.py:1-17)."""
from hetu_galvatron_b200 import __version__  # noqa: F401

from ._submodules import install as _install_submodules  # noqa: E402

_install_submodules()
