"""The model packages of the reference under their import paths.

Programs written against the reference import, per model directory (e.g. galvatron/models/llama_hf/train_dist.py:1-20,
train_dist_random.py:1-20, profiler.py, search_dist.py):

    from galvatron.models.llama_hf.LlamaModel_hybrid_parallel import get_llama_config, llama_model_hp, get_runtime_profiler
    from galvatron.models.llama_hf.LlamaModel_checkpoint import save_llama_module
    from galvatron.models.llama_hf.arguments import model_args, layernum_arg_names
    from galvatron.models.llama_hf.dataloader import DataLoaderForLlama, random_collate_fn
    from galvatron.models.llama_hf.meta_configs import model_name, model_layer_configs

``install(root)`` registers one module tree per reference directory (``llama_hf, llama_fa, gpt_hf, gpt_fa, bert_hf,
vit_hf, T5, swin``) below the package ``root`` with these names bound to this package's implementations. The ``galvatron``
import alias calls it for ``galvatron.models``; nothing is copied, every name is a thin binding.
"""
from __future__ import annotations

import sys
import types
from typing import Dict

# reference directory -> (family name here, prefix of its module files, short name in function names, dataset class name)
DIRECTORIES = {
    "llama_hf": ("llama_hf", "Llama", "llama", "DataLoaderForLlama"),
    "llama_fa": ("llama_fa", "Llama", "llama", "DataLoaderForLlama"),
    "gpt_hf": ("gpt_hf", "GPT", "gpt", "DataLoaderForGPT"),
    "gpt_fa": ("gpt_fa", "GPT", "gpt", "DataLoaderForGPT"),
    "bert_hf": ("bert_hf", "Bert", "bert", "DataLoaderForBert"),
    "vit_hf": ("vit_hf", "ViT", "vit", "DataLoaderForViT"),
    "T5": ("t5", "T5", "t5", "DataLoaderForT5"),
    "swin": ("swin", "Swin", "swin", "DataLoaderForSwin"),
}


def _module(name: str, doc: str, names: Dict[str, object]) -> types.ModuleType:
    mod = types.ModuleType(name, doc)
    mod.__dict__.update(names)
    mod.__all__ = sorted(names)
    sys.modules[name] = mod
    return mod


def _family_modules(root: str, directory: str) -> types.ModuleType:
    from ..core import construct_hybrid_parallel_model_api, get_hybrid_parallel_configs_api
    from ..core.checkpoint import load_model, save_model
    from . import dataloader as data
    from . import model_name_and_layer_configs
    from .api import family_api
    from .arguments import base_family, config_from_args, layernum_arg_names, make_model_args
    from .runner import get_runtime_profiler as _runtime_profiler

    family, prefix, short, dataset = DIRECTORIES[directory]
    base = base_family(family)
    get_config, model_hp, model_info = family_api(family)
    pkg = "%s.%s" % (root, directory)

    def get_runtime_profiler(args, path, config, start_iter=10, end_iter=20):
        return _runtime_profiler(args, path, config, family, start_iter=start_iter, end_iter=end_iter)

    def save_module(save_path, model, optimizer=None, opt_param_scheduler=None, iter_num=0, args=None):
        """Distributed checkpoint of iteration ``iter_num`` (reference signature: ``save_<family>_module(save_path, model,
        optimizer, opt_param_scheduler, iter_num, args)``)."""
        save_model(model, save_path, family, iter_num, optimizer=optimizer)

    def load_module(load_path, model, iter_num=None, args=None):
        load_model(model, load_path, family, iteration=iter_num)

    def model_name(config, args=None):
        return model_name_and_layer_configs(family, config, args)[0]

    def model_layer_configs(config):
        return model_name_and_layer_configs(family, config, None)[1]

    def set_model_config(config, args, overwrite_args=True):
        """The configuration that the flags in ``args`` describe (``config`` is accepted for the reference's call shape)."""
        return get_config(args, overwrite_args=overwrite_args)

    def config_from_meta(model_type: str):
        """The size table entry ``model_type`` as a ModelConfig."""
        import torch

        from . import build_model_specs

        return build_model_specs(base, dtype=torch.bfloat16, model_size=model_type)[0]

    def seqlen_arg_names():
        if base == "t5":
            return ["encoder_seq_length", "decoder_seq_length"]
        return [] if base in ("vit", "swin") else ["seq_length"]

    def get_batch(data_iterator):
        """The next batch of this rank in the reference's shape ``input, keyword arguments incl. the labels, loss function``
        (models/llama_hf/dataloader.py:138-164), from an iterator that yields ``(input, labels[, extras])``."""
        out = next(data_iterator)
        if len(out) == 3 and isinstance(out[1], dict):
            return out                                   # already in the reference's shape
        extras = dict(out[2]) if len(out) > 2 else {}
        return out[0], dict(extras, labels=out[1]), loss_func

    def get_train_valid_test_data_iterators(args=None, cfg=None, model=None):
        """(train, validation, test) iterators over the token files of ``--data-path``. Without arguments, as the
        reference's programs call it, it uses what ``set_megatron_args_for_dataset(args, model, ...)`` was given."""
        from .. import core

        ctx = core.DATASET_CONTEXT
        args = args if args is not None else ctx.get("args")
        model = model if model is not None else ctx.get("model")
        if args is None or model is None:
            raise RuntimeError("call set_megatron_args_for_dataset(args, model, ...) first, or pass args, cfg and model")
        return data.get_train_valid_test_data_iterators(args, cfg if cfg is not None else model.cfg, model)

    def loss_func(*_unused, **_kw):
        """Kept for the call shape ``forward_backward(batch, iter, profiler, loss_func=...)``: the loss is computed inside the
        last block of the model (fused with the head GEMM), so there is nothing for a user function to add."""
        return None

    dataset_cls, own_collate = data.DATASETS[base]

    def collate(batch):
        """The reference's batch shape: ``(input, keyword arguments of forward_backward incl. the labels, loss function)``."""
        out = own_collate(batch)
        extras = dict(out[2]) if len(out) > 2 else {}
        if base == "t5":
            extras["dec_tokens"] = extras.pop("decoder_input_ids")
            return out[0], dict(extras, dec_labels=out[1]), None
        return out[0], dict(extras, labels=out[1]), None

    loader_names = {dataset: dataset_cls, "random_collate_fn": collate, "get_batch": get_batch, "loss_func": loss_func,
                    "get_train_valid_test_data_iterators": get_train_valid_test_data_iterators}
    if base == "bert":
        loader_names["random_collate_fn_bert"] = collate
    if base == "vit":
        loader_names["vit_collate_fn"] = collate
    hp_names = {"get_%s_config" % short: get_config, "%s_model_hp" % short: model_hp, "%sModelInfo" % prefix: model_info,
                "get_runtime_profiler": get_runtime_profiler, "construct_hybrid_parallel_model": construct_hybrid_parallel_model_api,
                "get_hybrid_parallel_configs": get_hybrid_parallel_configs_api}
    subs = {
        "%sModel_hybrid_parallel" % prefix: hp_names,
        "%sModel_checkpoint" % prefix: {"save_%s_module" % short: save_module, "load_%s_module" % short: load_module},
        "arguments": {"model_args": make_model_args(family), "layernum_arg_names": lambda: layernum_arg_names(family),
                      "seqlen_arg_names": seqlen_arg_names},
        "dataloader": loader_names,
        "meta_configs": {"model_name": model_name, "model_layer_configs": model_layer_configs, "set_model_config": set_model_config,
                         "config_from_meta": config_from_meta, "config_from_args": lambda args, dtype: config_from_args(family, args, dtype)},
    }
    top = dict(hp_names)
    package = _module(pkg, "Names of the reference's galvatron/models/%s, bound to hetu_galvatron_b200." % directory, top)
    package.__path__ = []                       # a package: its submodules are the entries registered below
    for sub, names in subs.items():
        setattr(package, sub, _module("%s.%s" % (pkg, sub), "galvatron/models/%s/%s" % (directory, sub), names))
    return package


def install(root: str) -> Dict[str, types.ModuleType]:
    """Register ``root.<directory>`` and its submodules for every model directory of the reference; returns the packages."""
    return {d: _family_modules(root, d) for d in DIRECTORIES}
