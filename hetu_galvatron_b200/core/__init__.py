"""Public facade, under the names a user of the reference imports from ``galvatron.core``
(galvatron/core/__init__.py:1-19): profilers, the model-construction API, the search engine, argument parsing.

    from hetu_galvatron_b200.core import (initialize_galvatron, get_hybrid_parallel_configs_api,
                                          construct_hybrid_parallel_model_api, GalvatronSearchEngine, ...)

Heavy submodules are imported on first attribute access so ``import hetu_galvatron_b200.core`` stays cheap.
"""
from __future__ import annotations

import importlib
from contextlib import contextmanager

_EXPORTS = {
    "ModelProfiler": ("..profiler.model_profiler", "ModelProfiler"),
    "HardwareProfiler": ("..profiler.hardware_profiler", "HardwareProfiler"),
    "RuntimeProfiler": ("..profiler.runtime_profiler", "RuntimeProfiler"),
    "GalvatronSearchEngine": ("..search", "GalvatronSearchEngine"),
    "initialize_galvatron": (".arguments", "initialize_galvatron"),
    "get_args": (".arguments", "get_args"),
    "get_optimizer_and_param_scheduler": (".optimizer", "get_optimizer_and_param_scheduler"),
    "clip_grad_norm": (".optimizer", "clip_grad_norm"),
    "HybridPlan": (".plan", "HybridPlan"),
    "GalvatronModel": (".hybrid_model", "GalvatronModel"),
    "ModuleSpec": (".hybrid_model", "ModuleSpec"),
    "construct_hybrid_parallel_model": (".hybrid_model", "construct_hybrid_parallel_model"),
    "save_model": (".checkpoint", "save_model"),
    "load_model": (".checkpoint", "load_model"),
    "Heartbeat": (".failure", "Heartbeat"),
    "RankFailure": (".failure", "RankFailure"),
    "guarded_step": (".failure", "guarded_step"),
    # runtime names of the reference (galvatron/core/runtime/__init__.py:1-4) and their counterparts here
    "ModelInfo": (".model_info", "ModelInfo"),
    "PipelineParallel": ("..parallel.pipeline", "PipelineParallel"),
    "PipeSequential": ("..parallel.pipeline", "StageModule"),
    "ParallelAttention": ("..models.transformer", "SelfAttention"),
    "ParallelMLP": ("..models.transformer", "MLP"),
    "gen_comm_groups": ("..parallel.mesh", "gen_comm_groups"),
    "mixed_precision_dtype": ("..utils.attr_utils", "mixed_precision_dtype"),
    "rgetattr": ("..utils.attr_utils", "rgetattr"),
    "rsetattr": ("..utils.attr_utils", "rsetattr"),
    "rhasattr": ("..utils.attr_utils", "rhasattr"),
    "galvatron_training_args": (".arguments", "galvatron_training_args"),
    "galvatron_profile_args": ("..profiler.arguments", "galvatron_profile_args"),
    "galvatron_profile_hardware_args": ("..profiler.arguments", "galvatron_profile_hardware_args"),
    "galvatron_search_args": ("..search.arguments", "galvatron_search_args"),
}

__all__ = sorted(list(_EXPORTS) + ["init_empty_weights", "get_hybrid_parallel_configs_api",
                                   "construct_hybrid_parallel_model_api", "set_megatron_args_for_dataset"])


def __getattr__(name: str):
    if name in _EXPORTS:
        mod, attr = _EXPORTS[name]
        value = getattr(importlib.import_module(mod, __name__), attr)
        globals()[name] = value
        return value
    raise AttributeError("module %r has no attribute %r" % (__name__, name))


@contextmanager
def init_empty_weights(include_buffers: bool = True):
    """Create modules without allocating their tensors (reference: galvatron/core/runtime/initialize.py:7-104, which
    patches ``register_parameter``; PyTorch's meta device gives the same effect) for user code that builds plain
    modules. This package's own blocks are built directly in sharded form on their device; inside this context they are
    built without initial values (``models.transformer.deferred_init``), to be filled by ``load_model`` -- what
    ``--initialize_on_meta 1 --load PATH`` does in the training programs."""
    import torch

    from ..models.transformer import deferred_init

    with torch.device("meta"), deferred_init():
        yield


def get_hybrid_parallel_configs_api(config, args, model_info=None, num_layers=None):
    """Plan of the run from the parsed flags: the strategy JSON named by ``--galvatron_config_path`` or the GLOBAL
    flags (``--pp_deg --global_tp_deg --sdp ...``); reference hybrid_parallel_config.py:17-158. Returns a ``HybridPlan``
    (``plan.as_runtime_dict()`` is the reference's dict form)."""
    from .plan import HybridPlan
    import torch.distributed as dist

    n = num_layers if num_layers is not None else getattr(config, "num_layers", None)
    world = dist.get_world_size() if dist.is_initialized() else 1
    path = getattr(args, "galvatron_config_path", None)
    if path:
        plan = HybridPlan.from_json(path, n, sequence_parallel=getattr(args, "sequence_parallel", False),
                                    pipeline_type=getattr(args, "pipeline_type", "pipedream_flush"),
                                    default_dp_type=getattr(args, "default_dp_type", "ddp"))
        if getattr(args, "global_train_batch_size", None):
            plan.global_bsz = plan.global_bsz or args.global_train_batch_size
        return _write_back(args, plan)
    plan = HybridPlan.from_global(n, world, pp_deg=args.pp_deg, global_tp_deg=args.global_tp_deg,
                                  global_cp_deg=getattr(args, "global_cp_deg", 1), sdp=getattr(args, "sdp", 0),
                                  global_checkpoint=getattr(args, "global_checkpoint", 0),
                                  global_bsz=args.global_train_batch_size, chunks=getattr(args, "chunks", -1),
                                  pipeline_type=getattr(args, "pipeline_type", "pipedream_flush"),
                                  default_dp_type=getattr(args, "default_dp_type", "ddp"),
                                  vocab_tp=getattr(args, "vocab_tp", 1), vocab_cp=getattr(args, "vocab_cp", 1),
                                  use_ulysses=getattr(args, "use_ulysses", False), embed_sdp=getattr(args, "embed_sdp", 0),
                                  sequence_parallel=getattr(args, "sequence_parallel", False))
    if getattr(args, "global_tp_consec", -1) == 0:
        # kept in the saved plan for the reference's tools; ranks of a tensor-parallel group are laid out consecutively
        # either way (every peer is equally near on one NVSwitch box)
        plan.tp_consecutive_flags = [0] * n
    return _write_back(args, plan)


def _write_back(args, plan):
    """The resolved plan is written back into ``args`` under the names the reference fills in
    (hybrid_parallel_config.py:36-41,60-84), which its programs read afterwards (``args.vocab_sp``, ``args.chunks`` ...)."""
    for name, value in (("global_train_batch_size", plan.global_bsz), ("chunks", plan.chunks), ("pp_deg", plan.pp_deg),
                        ("vocab_tp", plan.vocab_tp), ("vocab_sp", plan.vocab_sp), ("vocab_cp", plan.vocab_cp),
                        ("pipeline_type", plan.pipeline_type), ("default_dp_type", plan.default_dp_type),
                        ("embed_sdp", plan.embed_sdp)):
        try:
            setattr(args, name, value)
        except AttributeError:          # a read-only namespace: the plan itself still carries every value
            pass
    return plan


def construct_hybrid_parallel_model_api(specs, config, args, plan, device=None, **kw):
    """Model assembly under the reference's entry-point name (hybrid_parallel_model.py:165-326). ``specs`` is the
    family's module list (``hetu_galvatron_b200.models.specs_for``) instead of a HuggingFace model to operate on."""
    import torch

    from .hybrid_model import construct_hybrid_parallel_model

    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    return construct_hybrid_parallel_model(config, plan, specs, device, impl=getattr(args, "comm_impl", "nccl"),
                                           async_grad_reduce=bool(getattr(args, "async_grad_reduce", 1)), **kw)


DATASET_CONTEXT = {}      # what the last set_megatron_args_for_dataset call was given: {"args": ..., "model": ...}


def set_megatron_args_for_dataset(args, hp_model, *groups):
    """Reference runtime/utils.py:67-98 points Megatron's globals at the embedding layer's groups (tensor / data / context
    parallel, passed after the model) so that its dataset code broadcasts batches correctly. Here the data iterator
    (``core.dataloader.build_token_iterator``) reads the rank's slice straight from ``hp_model.batch_slice()``, so the
    groups are not needed; the call restores the iteration counter of a resumed run, fills the batch-size names that
    Megatron-style loops read, and remembers ``args`` and the model for the argument-less
    ``get_train_valid_test_data_iterators()`` of the reference's programs."""
    if getattr(args, "distributed_checkpoint", False) and getattr(args, "load", None):
        args.iteration = getattr(args, "load_iteration", 0)
    else:
        args.iteration = 0
    if getattr(args, "global_batch_size", None) is None:
        args.global_batch_size = getattr(args, "global_train_batch_size", None)
    DATASET_CONTEXT.update(args=args, model=hp_model)
    return args
