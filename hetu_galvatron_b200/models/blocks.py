"""Stage-level wrappers with the uniform ``forward(x, ctx)`` signature the stage runner expects
(the reference's *Embeddings_ / *Layers_ / *PreNorm_ / *Cls_ wrappers, e.g.
galvatron/models/llama_hf/LlamaModel_sequential.py:28-187)."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ..parallel.reshard import Layout, seq_positions
from .transformer import (BatchCtx, FinalNorm, LayerStrategy, LMHead, ModelConfig, TokenEmbedding, TransformerLayer)


def _layout(st: LayerStrategy) -> Layout:
    return Layout(tp=st.tp, cp=st.cp, seq_sharded=st.sp in ("megatron", "ulysses") and st.tp > 1)


def local_positions(st: LayerStrategy, seq: int, device) -> Optional[torch.Tensor]:
    """Global positions of the sequence rows this rank holds when the module slices the sequence itself
    (Ulysses and context parallelism); None when it sees the full sequence or Megatron-SP scatters it."""
    if st.cp == 1 and not (st.sp == "ulysses" and st.tp > 1):
        return None
    lay = Layout(tp=st.tp, cp=st.cp, seq_sharded=st.sp == "ulysses" and st.tp > 1)
    return seq_positions(lay, st.cp_rank * st.tp + st.tp_rank, seq).to(device)


class EmbedBlock(nn.Module):
    def __init__(self, cfg: ModelConfig, st: LayerStrategy, device):
        super().__init__()
        self.cfg, self.st = cfg, st
        self.embed = TokenEmbedding(cfg, st, device)
        if cfg.tie_embeddings:
            self.tie_key = "wte"

    def forward(self, ids_bs: torch.Tensor, ctx: BatchCtx):
        ids = ids_bs.t().contiguous()
        ctx.batch = ids.shape[1]
        pos = local_positions(self.st, ids.shape[0], ids.device)
        if pos is not None:
            ids = ids[pos].contiguous()
            ctx.positions = pos
        h = self.embed(ids, ctx)
        ctx.positions = None
        return h


class LayerBlock(nn.Module):
    def __init__(self, cfg: ModelConfig, st: LayerStrategy, layer_idx: int, device, **kw):
        super().__init__()
        self.layer = TransformerLayer(cfg, st, layer_idx, device, **kw)

    def forward(self, h, ctx: BatchCtx):
        return self.layer(h, ctx)


class NormBlock(nn.Module):
    def __init__(self, cfg: ModelConfig, st: LayerStrategy, device):
        super().__init__()
        self.norm = FinalNorm(cfg, st, device)

    def forward(self, h, ctx: BatchCtx):
        return self.norm(h, ctx)


class HeadBlock(nn.Module):
    def __init__(self, cfg: ModelConfig, st: LayerStrategy, device, tied: Optional[nn.Parameter] = None,
                 fp32_logits: bool = False):
        super().__init__()
        self.cfg, self.st = cfg, st
        self.head = LMHead(cfg, st, device, tied=tied, fp32_logits=fp32_logits)
        if cfg.tie_embeddings:
            self.tie_key = "wte"

    def forward(self, h, ctx: BatchCtx):
        labels = ctx.labels.t().contiguous()            # [s, b]
        pos = local_positions(self.st, labels.shape[0], labels.device)
        if pos is not None:
            labels = labels[pos].contiguous()
        saved = ctx.labels
        ctx.labels = labels
        mask = ctx.extra.get("loss_mask")
        if mask is not None:
            m = mask.t().contiguous()
            ctx.loss_mask = m[pos].contiguous() if pos is not None else m
        loss = self.head(h, ctx)
        ctx.labels = saved
        ctx.loss_mask = None
        return loss
