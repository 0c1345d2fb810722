"""BERT encoder family (post-LN blocks, word + position + token-type embeddings, masked-LM head).

Reference: galvatron/models/bert_hf/ (BertModel_sequential.py:250 module types ``embed, bert_enc x L, mlm_head``;
post-LN BertModel_tensor_parallel.py:31-57)."""
from __future__ import annotations

import json
import os
from typing import List

import torch
import torch.nn as nn

from ..core.hybrid_model import ModuleSpec
from ..ops import autograd as A
from .blocks import EmbedBlock, HeadBlock, LayerBlock
from .transformer import BatchCtx, LayerStrategy, ModelConfig, Norm, _det_normal

META_DIR = os.path.join(os.path.dirname(__file__), "meta_configs")
BERT_SIZES = ["bert-base", "bert-large", "bert-huge-32", "bert-huge-48"]


def bert_config(model_size: str = "bert-base", seq_length=None, dtype=torch.bfloat16, **overrides) -> ModelConfig:
    with open(os.path.join(META_DIR, model_size + ".json")) as fp:
        meta = json.load(fp)
    cfg = ModelConfig(hidden_size=meta["hidden_size"], num_heads=meta["num_attention_heads"],
                      ffn_hidden_size=meta["intermediate_size"], num_layers=meta["num_hidden_layers"],
                      vocab_size=meta["vocab_size"], seq_length=seq_length or meta["max_position_embeddings"], norm="layer",
                      norm_eps=meta.get("layer_norm_eps", 1e-12), act="gelu", pos="learned", bias=True, causal=False,
                      post_ln=True, tie_embeddings=True, type_vocab_size=meta.get("type_vocab_size", 2), dtype=dtype,
                      model_type="bert", make_vocab_size_divisible_by=128)
    for k, v in overrides.items():
        if v is not None:
            setattr(cfg, k, v)
    cfg.__post_init__()
    return cfg


class MLMHeadBlock(nn.Module):
    """transform (dense + GELU + LayerNorm) -> decoder tied to the word embedding -> masked-LM cross entropy."""

    def __init__(self, cfg: ModelConfig, st: LayerStrategy, device, tied=None):
        super().__init__()
        self.dense = nn.Parameter(_det_normal((cfg.hidden_size, cfg.hidden_size), cfg.init_std, 17, device, cfg.dtype))
        self.dense_bias = nn.Parameter(torch.zeros(cfg.hidden_size, dtype=cfg.dtype, device=device))
        sp = st.sp == "megatron" and st.tp > 1
        for p in (self.dense, self.dense_bias):
            p.tp_duplicate = st.weight_tp > 1
            p.sequence_parallel = sp
        self.ln = Norm(cfg, device, sp, st.weight_tp > 1)
        self.head = HeadBlock(cfg, st, device, tied=tied)
        self.tie_key = "wte"

    def forward(self, h, ctx: BatchCtx):
        x = A.linear(h, self.dense, self.dense_bias)
        x = self.ln(A.gelu(x))
        return self.head(x, ctx)


def bert_specs(cfg: ModelConfig) -> List[ModuleSpec]:
    shared = {}

    def build_embed(st, dev):
        blk = EmbedBlock(cfg, st, dev)
        shared["wte"] = blk.embed.wte
        return blk

    specs = [ModuleSpec("bert_embeddings", "embed", build_embed, None, "embed")]
    for i in range(cfg.num_layers):
        specs.append(ModuleSpec("bert_encoder_layer_%d" % i, "layer", (lambda st, dev, i=i: LayerBlock(cfg, st, i, dev)), i, "bert_enc"))
    specs.append(ModuleSpec("cls_predictions", "cls", lambda st, dev: MLMHeadBlock(cfg, st, dev, tied=shared.get("wte")), None, "mlm_head"))
    return specs


def model_name(cfg: ModelConfig) -> str:
    return "hidden%d_head%d_seqlen%d" % (cfg.hidden_size, cfg.num_heads, cfg.seq_length)


def model_layer_configs(cfg: ModelConfig):
    return [{"hidden_size": cfg.hidden_size, "seq_len": cfg.seq_length, "layer_num": cfg.num_layers}]


# entry points under the reference's names (models/api.py)
from .api import family_api  # noqa: E402

get_bert_config, bert_model_hp, BertModelInfo = family_api("bert")
