"""Submodule paths of the reference package, resolved on import.

``from galvatron.core.search_engine.cost_model import TimeCostModel`` and the like name modules of the reference's tree
(galvatron/core/{profiler,runtime,search_engine}/*.py, galvatron/utils/*.py). This finder answers those names with a module
that carries the public names of the counterpart(s) in ``hetu_galvatron_b200``; nothing is imported before it is asked for.
"""
import importlib
import importlib.abc
import importlib.util
import sys

H = "hetu_galvatron_b200."
# reference module -> the module(s) here whose names it offers (later entries win on a clash); "" marks a pure package
TABLE = {
    "galvatron.core.arguments": [H + "core.arguments"],
    "galvatron.core.search_engine": [H + "search"],
    "galvatron.core.search_engine.search_engine": [H + "search.search_engine"],
    "galvatron.core.search_engine.cost_model": [H + "search.cost_model"],
    "galvatron.core.search_engine.cost_model_args": [H + "search.cost_model_args"],
    "galvatron.core.search_engine.dynamic_programming": [H + "search.dynamic_programming"],
    "galvatron.core.search_engine.arguments": [H + "search.arguments"],
    "galvatron.core.search_engine.utils": [H + "search.log_utils"],
    "galvatron.core.profiler": [H + "profiler.model_profiler", H + "profiler.hardware_profiler", H + "profiler.runtime_profiler"],
    "galvatron.core.profiler.model_profiler": [H + "profiler.model_profiler"],
    "galvatron.core.profiler.hardware_profiler": [H + "profiler.hardware_profiler"],
    "galvatron.core.profiler.runtime_profiler": [H + "profiler.runtime_profiler"],
    "galvatron.core.profiler.arguments": [H + "profiler.arguments"],
    "galvatron.core.profiler.utils": [H + "profiler.utils"],
    "galvatron.core.runtime": [H + "core"],
    "galvatron.core.runtime.arguments": [H + "core.arguments"],
    "galvatron.core.runtime.hybrid_parallel_config": [H + "core.plan", H + "core"],
    "galvatron.core.runtime.hybrid_parallel_model": [H + "core.hybrid_model", H + "core"],
    "galvatron.core.runtime.comm_groups": [H + "parallel.mesh"],
    "galvatron.core.runtime.redistribute": [H + "parallel.reshard"],
    "galvatron.core.runtime.initialize": [H + "core"],
    "galvatron.core.runtime.dataloader": [H + "core.dataloader"],
    "galvatron.core.runtime.utils": [H + "core.optimizer", H + "utils.attr_utils", H + "core"],
    "galvatron.tools": [],
    "galvatron.tools.checkpoint_convert_h2g": [H + "tools.checkpoint_convert_h2g"],
    "galvatron.tools.checkpoint_convert_g2h": [H + "tools.checkpoint_convert_g2h"],
    "galvatron.utils.config_utils": [H + "utils.config_utils"],
    "galvatron.utils.memory_utils": [H + "utils.memory_utils"],
    "galvatron.utils.strategy_utils": [H + "utils.strategy_utils"],
    "galvatron.utils.training_utils": [H + "utils.training_utils"],
}
PACKAGES = {"galvatron.core.search_engine", "galvatron.core.profiler", "galvatron.core.runtime", "galvatron.tools"}


class _Finder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, name, path=None, target=None):
        if name in TABLE:
            return importlib.util.spec_from_loader(name, self, is_package=name in PACKAGES)
        return None

    def create_module(self, spec):
        return None                      # a fresh module; exec_module fills it

    def exec_module(self, module):
        sources = [importlib.import_module(t) for t in TABLE[module.__name__]]
        module.__doc__ = "Names of %s under the reference's path %s." % (", ".join(TABLE[module.__name__]), module.__name__)
        for src in sources:
            exported = getattr(src, "__all__", None) or [k for k in vars(src) if not k.startswith("_")]
            for k in exported:
                try:
                    module.__dict__[k] = getattr(src, k)
                except AttributeError:
                    pass
        lazy = [s for s in sources if hasattr(s, "__getattr__")]

        def __getattr__(name, _lazy=lazy):          # modules here that resolve some names lazily keep doing so
            for s in _lazy:
                try:
                    return getattr(s, name)
                except AttributeError:
                    continue
            raise AttributeError("module %r has no attribute %r" % (module.__name__, name))

        module.__getattr__ = __getattr__


def install() -> None:
    if not any(isinstance(f, _Finder) for f in sys.meta_path):
        sys.meta_path.append(_Finder())
