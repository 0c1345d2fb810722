"""GPT-2 style decoder family (LayerNorm, learned positions, GELU MLP with biases, tied embedding / head).

Reference: galvatron/models/gpt_hf/ (GPTModel_sequential.py:233-248 module types ``embed, gpt_dec x L, norm, cls``;
learned positions GPTModel_tensor_parallel.py:106-117; tied head GPTModel_hybrid_parallel.py:42; vocabulary padded to a
multiple of 128, meta_configs/config_utils.py:77-82)."""
from __future__ import annotations

import json
import os
from typing import List

import torch

from ..core.hybrid_model import ModuleSpec
from .blocks import EmbedBlock, HeadBlock, LayerBlock, NormBlock
from .transformer import ModelConfig

META_DIR = os.path.join(os.path.dirname(__file__), "meta_configs")
GPT_SIZES = ["gpt-0.3b", "gpt-1.5b", "gpt-2.7b", "gpt-6.7b"]


def gpt_config(model_size: str = "gpt-1.5b", seq_length=None, dtype=torch.bfloat16, **overrides) -> ModelConfig:
    if isinstance(model_size, dict):          # the size table entry itself (the reference takes either)
        meta = dict(model_size)
    else:
        with open(os.path.join(META_DIR, model_size + ".json")) as fp:
            meta = json.load(fp)
    cfg = ModelConfig(hidden_size=meta["n_embd"], num_heads=meta["n_head"], ffn_hidden_size=meta.get("n_inner") or 4 * meta["n_embd"],
                      num_layers=meta["n_layer"], vocab_size=meta["vocab_size"], seq_length=seq_length or meta["n_positions"],
                      norm="layer", norm_eps=meta.get("layer_norm_epsilon", 1e-5), act="gelu", pos="learned", bias=True,
                      causal=True, tie_embeddings=True, dtype=dtype, model_type="gpt", make_vocab_size_divisible_by=128)
    for k, v in overrides.items():
        if v is not None:
            setattr(cfg, k, v)
    cfg.__post_init__()
    return cfg


def gpt_specs(cfg: ModelConfig, fp32_logits: bool = False) -> List[ModuleSpec]:
    shared = {}

    def build_embed(st, dev):
        blk = EmbedBlock(cfg, st, dev)
        shared["wte"] = blk.embed.wte
        return blk

    def build_head(st, dev):
        return HeadBlock(cfg, st, dev, tied=shared.get("wte") if cfg.tie_embeddings else None, fp32_logits=fp32_logits)

    specs = [ModuleSpec("transformer_embedding", "embed", build_embed, None, "embed")]
    for i in range(cfg.num_layers):
        specs.append(ModuleSpec("transformer_h_%d" % i, "layer", (lambda st, dev, i=i: LayerBlock(cfg, st, i, dev)), i, "gpt_dec"))
    specs.append(ModuleSpec("transformer_ln_f", "norm", lambda st, dev: NormBlock(cfg, st, dev), None, "norm"))
    specs.append(ModuleSpec("lm_head", "cls", build_head, None, "cls"))
    return specs


def model_name(cfg: ModelConfig) -> str:
    return "hidden%d_head%d_seqlen%d" % (cfg.hidden_size, cfg.num_heads, cfg.seq_length)


def model_layer_configs(cfg: ModelConfig):
    return [{"hidden_size": cfg.hidden_size, "seq_len": cfg.seq_length, "layer_num": cfg.num_layers}]


# entry points under the reference's names (models/api.py)
from .api import family_api  # noqa: E402

get_gpt_config, gpt_model_hp, GPTModelInfo = family_api("gpt")
