"""Llama / Qwen-style decoder family (RMSNorm, RoPE, SwiGLU, GQA, untied head).

Reference: galvatron/models/llama_hf/ (LlamaModel_sequential.py:201-216 module types
``embed, gpt_dec x L, norm, cls``; meta_configs/config_utils.py:22-125 for the size table and names)."""
from __future__ import annotations

import json
import os
from typing import List

import torch

from ..core.hybrid_model import ModuleSpec
from .blocks import EmbedBlock, HeadBlock, LayerBlock, NormBlock
from .transformer import ModelConfig

META_DIR = os.path.join(os.path.dirname(__file__), "meta_configs")

LLAMA_SIZES = ["llama-0.3b", "llama-7b", "llama-13b", "llama-30b", "llama2-70b", "qwen2.5-1.5b", "qwen2.5-3b",
               "qwen2.5-7b", "qwen2.5-72b"]


def _ffn_from_multiple_of(dim: int, multiple_of: int) -> int:
    hidden = int(2 * (4 * dim) / 3)
    return multiple_of * ((hidden + multiple_of - 1) // multiple_of)


def llama_config(model_size: str = "llama-7b", seq_length: int | None = None, dtype=torch.bfloat16, **overrides) -> ModelConfig:
    if isinstance(model_size, dict):          # the size table entry itself (the reference takes either, config_utils.py:22-30)
        meta = dict(model_size)
    else:
        with open(os.path.join(META_DIR, model_size + ".json")) as fp:
            meta = json.load(fp)
    ffn = meta.get("ffn_dim") or _ffn_from_multiple_of(meta["dim"], meta.get("multiple_of", 256))
    cfg = ModelConfig(hidden_size=meta["dim"], num_heads=meta["n_heads"], num_kv_heads=meta.get("n_kv_heads", meta["n_heads"]),
                      ffn_hidden_size=ffn, num_layers=meta["n_layers"], vocab_size=meta["vocab_size"],
                      seq_length=seq_length or meta.get("n_positions", 2048), norm="rms", norm_eps=meta.get("norm_eps", 1e-5),
                      act="swiglu", pos="rope", rope_base=meta.get("rope_theta", 10000.0), bias=False, causal=True,
                      tie_embeddings=False, dtype=dtype, model_type="llama")
    for k, v in overrides.items():
        if v is not None:
            setattr(cfg, k, v)
    cfg.__post_init__()
    return cfg


def llama_specs(cfg: ModelConfig, fp32_logits: bool = False) -> List[ModuleSpec]:
    specs = [ModuleSpec("model_embed_tokens", "embed", lambda st, dev: EmbedBlock(cfg, st, dev), None, "embed")]
    for i in range(cfg.num_layers):
        specs.append(ModuleSpec("model_layers_%d" % i, "layer",
                                (lambda st, dev, i=i: LayerBlock(cfg, st, i, dev)), i, "gpt_dec"))
    specs.append(ModuleSpec("model_norm", "norm", lambda st, dev: NormBlock(cfg, st, dev), None, "norm"))
    specs.append(ModuleSpec("lm_head", "cls", lambda st, dev: HeadBlock(cfg, st, dev, fp32_logits=fp32_logits), None, "cls"))
    return specs


def model_name(cfg: ModelConfig) -> str:
    return "hidden%d_head%d_seqlen%d" % (cfg.hidden_size, cfg.num_heads, cfg.seq_length)


def model_layer_configs(cfg: ModelConfig):
    return [{"hidden_size": cfg.hidden_size, "seq_len": cfg.seq_length, "layer_num": cfg.num_layers}]


# entry points under the reference's names (models/api.py)
from .api import family_api  # noqa: E402

get_llama_config, llama_model_hp, LlamaModelInfo = family_api("llama")
