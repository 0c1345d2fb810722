"""Per-family entry points under the reference's names.

Every model directory of the reference exports ``get_<family>_config(args)``, ``<family>_model_hp(config, args)`` and a
``<Family>ModelInfo`` class (e.g. galvatron/models/llama_hf/LlamaModel_hybrid_parallel.py:44-84,
LlamaModel_sequential.py:201-216; used as ``config = get_llama_config(args); model = llama_model_hp(config, args)`` in
models/llama_hf/train_dist.py:24-41). ``family_api`` builds the three for a family; each family module binds them to
its own names, so user code that followed the reference keeps its shape:

    from hetu_galvatron_b200.models.llama import get_llama_config, llama_model_hp
    args = initialize_galvatron(model_args, mode="train_dist")
    config = get_llama_config(args)
    model = llama_model_hp(config, args)
"""
from __future__ import annotations

import torch


def family_api(family: str):
    def get_config(args, overwrite_args: bool = True):
        """ModelConfig from ``--model_size`` and the manual-override flags."""
        from .arguments import config_from_args

        dtype = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}[getattr(args, "mixed_precision", "bf16")]
        cfg, _ = config_from_args(family, args, dtype)
        if overwrite_args:
            for flag, value in (("hidden_size", cfg.hidden_size), ("num_hidden_layers", cfg.num_layers),
                                ("num_attention_heads", cfg.num_heads), ("seq_length", cfg.seq_length),
                                ("vocab_size", cfg.vocab_size)):
                setattr(args, flag, value)      # unconditionally, as the reference's overwrite_model_args does
        return cfg

    def model_hp(config, args):
        """The hybrid-parallel model of this rank (a ``GalvatronModel``) for ``config`` under the plan in ``args``."""
        from ..core import construct_hybrid_parallel_model_api, get_hybrid_parallel_configs_api
        from . import specs_for

        specs = specs_for(family, config, fp32_logits=getattr(args, "entropy_in_fp32", False))
        n_layers = len([s for s in specs if s.layer_index is not None])
        plan = get_hybrid_parallel_configs_api(config, args, num_layers=n_layers)
        model = construct_hybrid_parallel_model_api(specs, config, args, plan)
        if getattr(args, "load", None):
            from ..core.checkpoint import load_model

            load_model(model, args.load, family, iteration=args.load_iteration if getattr(args, "distributed_checkpoint", False) else None,
                       allow_plan_change=bool(getattr(args, "allow_plan_change", 0)))
        return model

    def model_info(config, args=None):
        from ..core.model_info import ModelInfo
        from . import specs_for

        return ModelInfo(config, specs_for(family, config))

    get_config.__name__, model_hp.__name__, model_info.__name__ = "get_%s_config" % family, "%s_model_hp" % family, "%sModelInfo" % family
    return get_config, model_hp, model_info
