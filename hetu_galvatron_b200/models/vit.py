"""Vision Transformer family (patch embedding as a GEMM, CLS token, learned positions, pre-LN, pooled classifier).

Reference: galvatron/models/vit_hf/ (ViTModel_sequential.py:52-59 patch embedding on rearranged patches, :116-178
pooler + column-parallel classifier + vocab-parallel CE over classes, :198-218 module types ``embed, vit_enc x L,
prenorm, cls``; sequence = (image / patch)^2 + 1)."""
from __future__ import annotations

import json
import os
from typing import List

import torch
import torch.nn as nn

from ..core.hybrid_model import ModuleSpec
from ..ops import autograd as A
from .blocks import LayerBlock, NormBlock
from .transformer import (_FULL_SEQUENCE, BatchCtx, LayerStrategy, ModelConfig, _det_normal, _ScatterSeq, _shard_rows,
                          hidden_dropout)

META_DIR = os.path.join(os.path.dirname(__file__), "meta_configs")
VIT_SIZES = ["vit-base", "vit-large", "vit-huge", "vit-xhuge"]


def vit_config(model_size: str = "vit-huge", dtype=torch.bfloat16, **overrides) -> ModelConfig:
    with open(os.path.join(META_DIR, model_size + ".json")) as fp:
        meta = json.load(fp)
    cfg = ModelConfig(hidden_size=meta["hidden_size"], num_heads=meta["num_attention_heads"],
                      ffn_hidden_size=meta["intermediate_size"], num_layers=meta["num_hidden_layers"], vocab_size=meta.get("num_labels", 1000),
                      norm="layer", norm_eps=meta.get("layer_norm_eps", 1e-12), act="gelu", pos="learned", bias=True, causal=False,
                      dtype=dtype, model_type="vit", image_size=meta.get("image_size", 224), patch_size=meta.get("patch_size", 16),
                      num_channels=meta.get("num_channels", 3), num_labels=meta.get("num_labels", 1000))
    for k, v in overrides.items():
        if v is not None:
            setattr(cfg, k, v)
    cfg.seq_length = (cfg.image_size // cfg.patch_size) ** 2 + 1
    cfg.vocab_size = cfg.num_labels
    cfg.__post_init__()
    return cfg


class ViTEmbedBlock(nn.Module):
    def __init__(self, cfg: ModelConfig, st: LayerStrategy, device):
        super().__init__()
        self.cfg, self.st = cfg, st
        k = cfg.num_channels * cfg.patch_size * cfg.patch_size
        self.k, self.k_pad = k, (k + 7) // 8 * 8          # GEMM reduction length padded to a 16-byte multiple
        w = _det_normal((cfg.hidden_size, k), cfg.init_std, 21, device, cfg.dtype)
        if self.k_pad != k:
            w = torch.cat([w, torch.zeros(cfg.hidden_size, self.k_pad - k, dtype=cfg.dtype, device=device)], 1)
        self.w_patch = nn.Parameter(w)
        self.b_patch = nn.Parameter(torch.zeros(cfg.hidden_size, dtype=cfg.dtype, device=device))
        self.cls_token = nn.Parameter(_det_normal((1, cfg.hidden_size), cfg.init_std, 22, device, cfg.dtype))
        self.pos = nn.Parameter(_det_normal((cfg.seq_length, cfg.hidden_size), cfg.init_std, 23, device, cfg.dtype))
        for p in self.parameters():
            p.tp_duplicate = st.weight_tp > 1

    def forward(self, pixels: torch.Tensor, ctx: BatchCtx):
        cfg = self.cfg
        b, c, H, W = pixels.shape
        p = cfg.patch_size
        gh, gw = H // p, W // p
        x = pixels.reshape(b, c, gh, p, gw, p).permute(2, 4, 0, 1, 3, 5).reshape(gh * gw * b, c * p * p)   # [(n, b), k]
        if self.k_pad != self.k:
            x = torch.nn.functional.pad(x, (0, self.k_pad - self.k))
        x = A.linear(x.to(cfg.dtype).contiguous(), self.w_patch, self.b_patch)                             # [n * b, h]
        n = gh * gw
        cls = self.cls_token.expand(b, cfg.hidden_size)
        h = torch.cat([cls, x], 0).view(n + 1, b, cfg.hidden_size) + self.pos.unsqueeze(1)
        ctx.batch = b
        h = h.reshape((n + 1) * b, cfg.hidden_size)
        if cfg.dropout > 0.0 and ctx.extra.get("rng") is not None:
            h = hidden_dropout(h, cfg.dropout, ctx, _FULL_SEQUENCE, 1)
        if self.st.sp == "megatron" and self.st.tp > 1:
            h = _ScatterSeq.apply(h, self.st.tp, self.st.tp_rank, self.st.pg())
        return h


class ViTHeadBlock(nn.Module):
    """CLS token -> pooler (dense + tanh) -> classifier (class-parallel over the vocab-tp group) -> cross entropy."""

    def __init__(self, cfg: ModelConfig, st: LayerStrategy, device):
        super().__init__()
        self.cfg, self.st = cfg, st
        t, r = st.weight_tp, st.tp_rank if st.weight_tp > 1 else 0
        self.w_pool = nn.Parameter(_det_normal((cfg.hidden_size, cfg.hidden_size), cfg.init_std, 24, device, cfg.dtype))
        self.b_pool = nn.Parameter(torch.zeros(cfg.hidden_size, dtype=cfg.dtype, device=device))
        for p in (self.w_pool, self.b_pool):
            p.tp_duplicate = t > 1
        full = _det_normal((cfg.num_labels, cfg.hidden_size), cfg.init_std, 25, device, cfg.dtype)
        self.class_start = r * (cfg.num_labels // t)
        self.w_cls = nn.Parameter(_shard_rows(full, t, r))

    def forward(self, h, ctx: BatchCtx):
        st, cfg = self.st, self.cfg
        if st.sp == "megatron" and st.tp > 1:
            from .transformer import _GatherSeq
            h = _GatherSeq.apply(h, st.tp, st.tp_rank, st.pg())
        cls = h[: ctx.batch]                                   # sequence-major: the first b rows are the CLS tokens
        pooled = torch.tanh(A.linear(cls.contiguous(), self.w_pool, self.b_pool))
        lcfg = A.LossCfg(vocab_start=self.class_start, group=st.pg() if st.weight_tp > 1 else None, mode="col")
        loss = A.lm_head_loss(pooled, self.w_cls, ctx.labels.reshape(-1), lcfg)
        return loss.mean()


def vit_specs(cfg: ModelConfig) -> List[ModuleSpec]:
    specs = [ModuleSpec("vit_embeddings", "embed", lambda st, dev: ViTEmbedBlock(cfg, st, dev), None, "embed")]
    for i in range(cfg.num_layers):
        specs.append(ModuleSpec("vit_encoder_layer_%d" % i, "layer", (lambda st, dev, i=i: LayerBlock(cfg, st, i, dev)), i, "vit_enc"))
    specs.append(ModuleSpec("vit_layernorm", "norm", lambda st, dev: NormBlock(cfg, st, dev), None, "prenorm"))
    specs.append(ModuleSpec("classifier", "cls", lambda st, dev: ViTHeadBlock(cfg, st, dev), None, "cls"))
    return specs


def model_name(cfg: ModelConfig) -> str:
    return "hidden%d_head%d" % (cfg.hidden_size, cfg.num_heads)


def model_layer_configs(cfg: ModelConfig):
    return [{"hidden_size": cfg.hidden_size, "seq_len": cfg.seq_length, "layer_num": cfg.num_layers}]


# entry points under the reference's names (models/api.py)
from .api import family_api  # noqa: E402

get_vit_config, vit_model_hp, ViTModelInfo = family_api("vit")
