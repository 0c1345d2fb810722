"""Swin Transformer family: four stages of windowed / shifted-window attention blocks with patch merging between them.

Reference: galvatron/models/swin/ (SwinModel_sequential.py:225-270: module types ``embed, (swin_enc x d_i
[, swin_downsample]) x 4, pooler, cls``; four layer types, each with its own sequence length
``(image / patch / 2^i)^2`` and hidden size ``embed_dim * 2^i``; SwinModel_tensor_parallel.py:14-41,101-191: window
partition / reverse, shifted-window mask, relative position bias). Here the patch merging that ends a stage is part of
that stage's last block, so the plan's layer list is exactly ``sum(depths)`` blocks; activations stay sequence-major
``[tokens * batch, hidden]`` with tokens in row-major (H, W) order. Tensor parallelism shards heads and the MLP;
sequence parallelism is not offered for this family (as in the reference, SwinModel_hybrid_parallel.py).
The projections, MLP and LayerNorm run on this package's kernels, and so does the windowed attention core: windows of
49 or 144 tokens are batch elements of the tcgen05 attention kernels, which add the relative-position bias (per head) and
the shifted-window mask (per window position) to the scores and return the bias gradient summed over the batch.
"""
from __future__ import annotations

import json
import os
from typing import List

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..core.hybrid_model import ModuleSpec
from ..ops import autograd as A
from .transformer import BatchCtx, LayerStrategy, ModelConfig, _det_normal, _shard_cols, _shard_rows

META_DIR = os.path.join(os.path.dirname(__file__), "meta_configs")
SWIN_SIZES = ["swin-huge-patch4-window7-224", "swin-large-patch4-window12-384", "swin-tiny-test"]


def swin_config(model_size: str = "swin-huge-patch4-window7-224", dtype=torch.bfloat16, **overrides) -> ModelConfig:
    with open(os.path.join(META_DIR, model_size + ".json")) as fp:
        meta = json.load(fp)
    depths = list(overrides.pop("depths", None) or meta["depths"])
    cfg = ModelConfig(hidden_size=meta["embed_dim"], num_heads=meta["num_heads"][0], ffn_hidden_size=meta["embed_dim"] * meta["mlp_ratio"],
                      num_layers=sum(depths), vocab_size=meta.get("num_labels", 1000), norm="layer",
                      norm_eps=meta.get("layer_norm_eps", 1e-5), act="gelu", pos="none", bias=True, causal=False, dtype=dtype,
                      model_type="swin", image_size=meta["image_size"], patch_size=meta["patch_size"],
                      num_channels=meta.get("num_channels", 3), num_labels=meta.get("num_labels", 1000))
    cfg.depths, cfg.embed_dim, cfg.stage_heads = depths, meta["embed_dim"], list(meta["num_heads"])
    cfg.window_size, cfg.mlp_ratio = meta["window_size"], meta["mlp_ratio"]
    # stochastic depth on the attention branch (SwinModel_tensor_parallel.py:63,76). Off unless asked for: ``"meta"`` takes
    # the model size's rate, which is what the training programs pass when --drop_path_rate is not given.
    cfg.drop_path_rate = 0.0
    for k, v in overrides.items():
        if v is not None:
            setattr(cfg, k, v)
    if cfg.drop_path_rate == "meta":
        cfg.drop_path_rate = float(meta.get("drop_path_rate", 0.0))
    cfg.drop_path_rate = float(cfg.drop_path_rate)
    assert 0.0 <= cfg.drop_path_rate < 1.0 and len(cfg.stage_heads) >= len(cfg.depths)
    cfg.stage_heads = [int(h) for h in cfg.stage_heads]
    cfg.hidden_size, cfg.num_heads, cfg.ffn_hidden_size = cfg.embed_dim, cfg.stage_heads[0], cfg.embed_dim * cfg.mlp_ratio
    cfg.num_layers = sum(cfg.depths)
    cfg.vocab_size = cfg.num_labels
    cfg.seq_length = (cfg.image_size // cfg.patch_size) ** 2
    for i in range(len(cfg.depths)):                       # per-stage sequence lengths, looked up by the pipeline engine
        setattr(cfg, "seq_length_stage%d" % i, stage_dims(cfg, i)[0] ** 2)
    setattr(cfg, "seq_length_stage%d" % len(cfg.depths), stage_dims(cfg, len(cfg.depths) - 1)[0] ** 2)
    return cfg


def stage_dims(cfg: ModelConfig, i: int):
    """(resolution, hidden, heads) of stage i."""
    return cfg.image_size // cfg.patch_size // (2 ** i), cfg.embed_dim * (2 ** i), cfg.stage_heads[i]


class _LN(nn.Module):
    def __init__(self, dim: int, cfg: ModelConfig, device, dup: bool):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=cfg.dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(dim, dtype=cfg.dtype, device=device))
        self.eps = cfg.norm_eps
        self.weight.tp_duplicate = self.bias.tp_duplicate = dup

    def forward(self, x):
        return A.layernorm(x, self.weight, self.bias, self.eps)


def _relative_index(ws: int) -> torch.Tensor:
    """[ws^2, ws^2] index into the (2 ws - 1)^2 relative-position table."""
    coords = torch.stack(torch.meshgrid(torch.arange(ws), torch.arange(ws), indexing="ij")).flatten(1)
    rel = (coords[:, :, None] - coords[:, None, :]).permute(1, 2, 0) + (ws - 1)
    return rel[..., 0] * (2 * ws - 1) + rel[..., 1]


def _shift_regions(res: int, ws: int, shift: int) -> torch.Tensor:
    """[windows, ws^2] region id of every token of every window of the shifted image: tokens of different regions were not
    neighbours before the cyclic shift and must not attend to each other."""
    img = torch.zeros(res, res, dtype=torch.int32)
    cnt = 0
    for hs in (slice(0, -ws), slice(-ws, -shift), slice(-shift, None)):
        for wsl in (slice(0, -ws), slice(-ws, -shift), slice(-shift, None)):
            img[hs, wsl] = cnt
            cnt += 1
    return img.view(res // ws, ws, res // ws, ws).permute(0, 2, 1, 3).reshape(-1, ws * ws).contiguous()


def _shift_mask(res: int, ws: int, shift: int) -> torch.Tensor:
    """[windows, ws^2, ws^2] additive mask (0 / -inf-like) separating the regions a cyclic shift glues together."""
    img = torch.zeros(res, res)
    cnt = 0
    for hs in (slice(0, -ws), slice(-ws, -shift), slice(-shift, None)):
        for wsl in (slice(0, -ws), slice(-ws, -shift), slice(-shift, None)):
            img[hs, wsl] = cnt
            cnt += 1
    win = img.view(res // ws, ws, res // ws, ws).permute(0, 2, 1, 3).reshape(-1, ws * ws)
    diff = win[:, None, :] - win[:, :, None]
    return torch.zeros_like(diff).masked_fill(diff != 0, -30000.0)


class _PermuteRows(torch.autograd.Function):
    """y = x[perm] for a permutation of the rows; the gradient is the same gather with the inverse permutation."""

    @staticmethod
    def forward(ctx, x, perm, inv):
        ctx.save_for_backward(perm, inv)
        return x.index_select(0, perm)

    @staticmethod
    def backward(ctx, dy):
        perm, inv = ctx.saved_tensors
        return dy.index_select(0, inv), None, None


class SwinLayerBlock(nn.Module):
    """One Swin block (W-MSA or SW-MSA + MLP); ``merge`` appends the 2x2 patch merging that ends a stage."""

    def __init__(self, cfg: ModelConfig, st: LayerStrategy, stage: int, index: int, layer_idx: int, merge: bool, device):
        super().__init__()
        self.cfg, self.st, self.merge = cfg, st, merge
        self.layer_idx = layer_idx
        self.res, C, heads = stage_dims(cfg, stage)
        self.C = C
        t, r = st.weight_tp, (st.tp_rank if st.weight_tp > 1 else 0)
        assert heads % t == 0, "swin stage %d has %d heads, not divisible by tp %d" % (stage, heads, t)
        self.heads_l, self.dh = heads // t, C // heads
        self.ws = min(cfg.window_size, self.res)
        self.shift = 0 if (index % 2 == 0 or self.ws == self.res) else self.ws // 2
        seed = 1000 + 17 * layer_idx
        dup = t > 1
        self.ln1, self.ln2 = _LN(C, cfg, device, dup), _LN(C, cfg, device, dup)
        wq, wk, wv = (_det_normal((C, C), cfg.init_std, seed + i, device, cfg.dtype) for i in range(3))
        self.wqkv = nn.Parameter(torch.cat([_shard_rows(wq, t, r), _shard_rows(wk, t, r), _shard_rows(wv, t, r)], 0))
        self.bqkv = nn.Parameter(torch.zeros(3 * C // t, dtype=cfg.dtype, device=device))
        self.wo = nn.Parameter(_shard_cols(_det_normal((C, C), cfg.init_std, seed + 3, device, cfg.dtype), t, r))
        self.bo = nn.Parameter(torch.zeros(C, dtype=cfg.dtype, device=device))
        table = _det_normal(((2 * self.ws - 1) ** 2, heads), cfg.init_std, seed + 4, device, cfg.dtype)
        self.rel_table = nn.Parameter(table[:, r * self.heads_l:(r + 1) * self.heads_l].contiguous())
        Fh = C * cfg.mlp_ratio
        self.w1 = nn.Parameter(_shard_rows(_det_normal((Fh, C), cfg.init_std, seed + 5, device, cfg.dtype), t, r))
        self.b1 = nn.Parameter(torch.zeros(Fh // t, dtype=cfg.dtype, device=device))
        self.w2 = nn.Parameter(_shard_cols(_det_normal((C, Fh), cfg.init_std, seed + 6, device, cfg.dtype), t, r))
        self.b2 = nn.Parameter(torch.zeros(C, dtype=cfg.dtype, device=device))
        self.bo.tp_duplicate = self.b2.tp_duplicate = dup
        self.register_buffer("rel_index", _relative_index(self.ws).to(device), persistent=False)
        self._perm_cache: dict = {}
        if self.shift:
            self.register_buffer("regions", _shift_regions(self.res, self.ws, self.shift).to(device), persistent=False)
        if merge:
            self.ln_merge = _LN(4 * C, cfg, device, dup)
            self.w_merge = nn.Parameter(_det_normal((2 * C, 4 * C), cfg.init_std, seed + 7, device, cfg.dtype))
            self.w_merge.tp_duplicate = dup

    def _window_rows(self, b: int, device):
        """Row permutation of the [tokens * batch, channels] activations that does the cyclic shift and the window
        partition in one gather: output row (image, window, token in window) <- input row (token, image); plus its
        inverse (window reverse and shift back)."""
        key = (b, str(device))
        cached = self._perm_cache.get(key)
        if cached is None:
            R, ws, nw = self.res, self.ws, self.res // self.ws
            bi, wy, wx, ty, tx = torch.meshgrid(torch.arange(b), torch.arange(nw), torch.arange(nw), torch.arange(ws),
                                                torch.arange(ws), indexing="ij")
            y = (wy * ws + ty + self.shift) % R
            x = (wx * ws + tx + self.shift) % R
            perm = ((y * R + x) * b + bi).reshape(-1)
            inv = torch.empty_like(perm)
            inv[perm] = torch.arange(perm.numel())
            cached = (perm.to(device), inv.to(device))
            self._perm_cache[key] = cached
        return cached

    def _attention(self, qkv: torch.Tensor, b: int) -> torch.Tensor:
        """Cyclic shift + window partition as ONE row gather, attention inside every window with the relative-position
        bias as an additive score term and the shifted-window mask as group ids (``A.biased_attention``: the tcgen05 attention kernels
        with batch elements = windows, q / k / v consumed as strided views of the gathered rows), window reverse + shift
        back as one gather with the inverse permutation."""
        R, ws, hl, dh = self.res, self.ws, self.heads_l, self.dh
        nw, S = R // ws, ws * ws
        perm, inv = self._window_rows(b, qkv.device)
        x = _PermuteRows.apply(qkv, perm, inv).view(b * nw * nw, S, 3, hl, dh)      # [windows, tokens, q|k|v, heads, dh]
        bias = self.rel_table[self.rel_index.view(-1)].view(S, S, hl).permute(2, 0, 1)
        regions = self.regions if self.shift else None  # [nw^2, S]: window w of every image uses regions[w]
        o = A.biased_attention(x[:, :, 0], x[:, :, 1], x[:, :, 2], bias, ids=regions)   # [windows, tokens, heads, dh]
        return _PermuteRows.apply(o.reshape(b * nw * nw * S, hl * dh), inv, perm)

    def _drop_path(self, y: torch.Tensor, ctx: BatchCtx, b: int) -> torch.Tensor:
        """Stochastic depth: the whole branch output of a sample is dropped with probability p and the survivors scaled by
        1 / (1 - p). The per-sample draw is a pure function of the step's dropout key and the layer, so tensor-parallel
        ranks agree on it and a recomputed forward repeats it."""
        p, key = self.cfg.drop_path_rate, ctx.extra.get("rng")
        seed = 0x9E3779B97F4A7C15
        for v in (*key, 7919 + self.layer_idx):
            seed = ((seed ^ (int(v) + 0x7F4A7C15)) * 0x100000001B3) % (1 << 63)
        g = torch.Generator(device=y.device)
        g.manual_seed(seed)
        keep = torch.empty(b, dtype=torch.float32, device=y.device).bernoulli_(1.0 - p, generator=g) * (1.0 / (1.0 - p))
        return (y.view(-1, b, y.shape[1]) * keep.to(y.dtype).view(1, b, 1)).view_as(y)

    def forward(self, h, ctx: BatchCtx):
        st, b = self.st, ctx.batch
        col = st.linear_cfg("col")
        row = st.linear_cfg("row")
        qkv = A.linear(self.ln1(h), self.wqkv, self.bqkv, cfg=col)
        if self.cfg.drop_path_rate > 0.0 and ctx.extra.get("rng") is not None:
            h = h + self._drop_path(A.linear(self._attention(qkv, b).contiguous(), self.wo, self.bo, cfg=row), ctx, b)
        else:
            h = A.linear(self._attention(qkv, b).contiguous(), self.wo, self.bo, residual=h, cfg=row)
        m = A.gelu(A.linear(self.ln2(h), self.w1, self.b1, cfg=col))
        h = A.linear(m, self.w2, self.b2, residual=h, cfg=row)
        if self.merge:
            R, C = self.res, self.C
            x = h.view(R // 2, 2, R // 2, 2, b, C).permute(0, 2, 4, 3, 1, 5).reshape((R // 2) ** 2 * b, 4 * C)   # (dw, dh, C) order
            h = A.linear(self.ln_merge(x.contiguous()), self.w_merge)
        return h


class SwinEmbedBlock(nn.Module):
    def __init__(self, cfg: ModelConfig, st: LayerStrategy, device):
        super().__init__()
        self.cfg = cfg
        k = cfg.num_channels * cfg.patch_size ** 2
        self.k, self.k_pad = k, (k + 7) // 8 * 8
        w = _det_normal((cfg.embed_dim, k), cfg.init_std, 31, device, cfg.dtype)
        if self.k_pad != k:
            w = torch.cat([w, torch.zeros(cfg.embed_dim, self.k_pad - k, dtype=cfg.dtype, device=device)], 1)
        self.w_patch = nn.Parameter(w)
        self.b_patch = nn.Parameter(torch.zeros(cfg.embed_dim, dtype=cfg.dtype, device=device))
        self.ln = _LN(cfg.embed_dim, cfg, device, st.weight_tp > 1)
        for p in (self.w_patch, self.b_patch):
            p.tp_duplicate = st.weight_tp > 1

    def forward(self, pixels, ctx: BatchCtx):
        cfg = self.cfg
        b, c, H, W = pixels.shape
        p = cfg.patch_size
        gh, gw = H // p, W // p
        x = pixels.reshape(b, c, gh, p, gw, p).permute(2, 4, 0, 1, 3, 5).reshape(gh * gw * b, c * p * p)
        if self.k_pad != self.k:
            x = F.pad(x, (0, self.k_pad - self.k))
        ctx.batch = b
        return self.ln(A.linear(x.to(cfg.dtype).contiguous(), self.w_patch, self.b_patch))


class SwinHeadBlock(nn.Module):
    """Final LayerNorm -> mean over tokens -> classifier (class-parallel over the vocab-tp group) -> cross entropy."""

    def __init__(self, cfg: ModelConfig, st: LayerStrategy, device):
        super().__init__()
        self.cfg, self.st = cfg, st
        _, C, _ = stage_dims(cfg, len(cfg.depths) - 1)
        self.C = C
        t, r = st.weight_tp, (st.tp_rank if st.weight_tp > 1 else 0)
        self.ln = _LN(C, cfg, device, t > 1)
        full = _det_normal((cfg.num_labels, C), cfg.init_std, 35, device, cfg.dtype)
        self.class_start = r * (cfg.num_labels // t)
        self.w_cls = nn.Parameter(_shard_rows(full, t, r))

    def forward(self, h, ctx: BatchCtx):
        b = ctx.batch
        pooled = self.ln(h).view(-1, b, self.C).float().mean(0).to(h.dtype)
        lcfg = A.LossCfg(vocab_start=self.class_start, group=self.st.pg() if self.st.weight_tp > 1 else None, mode="col")
        return A.lm_head_loss(pooled.contiguous(), self.w_cls, ctx.labels.reshape(-1), lcfg).mean()


def swin_specs(cfg: ModelConfig) -> List[ModuleSpec]:
    specs = [ModuleSpec("swin_embeddings", "embed", lambda st, dev: SwinEmbedBlock(cfg, st, dev), None, "embed")]
    layer = 0
    last = len(cfg.depths) - 1
    for i, d in enumerate(cfg.depths):
        for j in range(d):
            merge = (j == d - 1 and i != last)
            sp = ModuleSpec("swin_encoder_%d_%d" % (i, j), "layer",
                            (lambda st, dev, i=i, j=j, layer=layer, merge=merge: SwinLayerBlock(cfg, st, i, j, layer, merge, dev)),
                            layer, "swin_enc", seq_attr="seq_length_stage%d" % i)
            sp.hidden_size = stage_dims(cfg, i)[1]
            specs.append(sp)
            layer += 1
    head = ModuleSpec("swin_classifier", "cls", lambda st, dev: SwinHeadBlock(cfg, st, dev), None, "cls",
                      seq_attr="seq_length_stage%d" % last)
    head.hidden_size = stage_dims(cfg, last)[1]
    specs.append(head)
    return specs


def model_name(cfg: ModelConfig) -> str:
    return "swin_embed%d_window%d_image%d" % (cfg.embed_dim, cfg.window_size, cfg.image_size)


def model_layer_configs(cfg: ModelConfig):
    return [{"hidden_size": stage_dims(cfg, i)[1], "seq_len": stage_dims(cfg, i)[0] ** 2, "layer_num": d}
            for i, d in enumerate(cfg.depths)]


# entry points under the reference's names (models/api.py)
from .api import family_api  # noqa: E402

get_swin_config, swin_model_hp, SwinModelInfo = family_api("swin")
