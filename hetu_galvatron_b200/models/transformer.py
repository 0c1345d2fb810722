"""Model-family-independent transformer building blocks.

One set of modules covers the decoder-only (GPT, Llama), encoder (BERT, ViT) and encoder-decoder (T5)
families of the reference's model zoo (galvatron/models/*/ *Model_tensor_parallel.py, *Model_sequential.py):
the family is a ``ModelConfig`` (norm kind, positional scheme, MLP kind, biases, causal mask, pre/post-LN),
the parallel layout of each layer is a ``LayerStrategy``.

Activations are sequence-major 2-D tensors ``[s_local * b_local, hidden]`` (token index = s * b + b_idx), so the
Megatron-SP all-gather / reduce-scatter along the sequence is a plain concatenation of rows and the attention
kernel reads q/k/v straight out of the packed projection through strides. Replaces
galvatron/core/runtime/tensor_parallel/transformer.py:82-166 (ParallelMLP) and :512-900 (ParallelAttention).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Optional

import torch
import torch.nn as nn

from ..ops import autograd as A
from ..ops import functional as Fn
from ..ops.gemm import RopeEpilogue
from ..parallel import collectives as C


@dataclass
class ModelConfig:
    hidden_size: int = 4096
    num_heads: int = 32
    num_kv_heads: Optional[int] = None
    ffn_hidden_size: int = 11008
    num_layers: int = 32
    vocab_size: int = 32000
    seq_length: int = 2048
    norm: str = "rms"            # rms | layer
    norm_eps: float = 1e-5
    act: str = "swiglu"          # swiglu | gelu
    pos: str = "rope"            # rope | learned | none
    rope_base: float = 10000.0
    bias: bool = False
    causal: bool = True
    post_ln: bool = False        # BERT: LayerNorm after the residual add
    tie_embeddings: bool = False
    init_std: float = 0.02
    dtype: torch.dtype = torch.bfloat16
    model_type: str = "llama"
    # vision
    image_size: int = 224
    patch_size: int = 16
    num_channels: int = 3
    num_labels: int = 1000
    # encoder-decoder
    num_decoder_layers: int = 0
    decoder_seq_length: Optional[int] = None     # None: the decoder runs at ``seq_length``
    # T5 relative position bias: 0 = none (what the reference's T5 runs, T5Model_tensor_parallel.py:13-14); 32 = the
    # published T5 models. Every self-attention layer then owns a [buckets, heads] table added to its scores.
    relative_attention_num_buckets: int = 0
    relative_attention_max_distance: int = 128
    type_vocab_size: int = 0
    dropout: float = 0.0
    attention_dropout: Optional[float] = None    # dropout of the attention probabilities; None = same as ``dropout``
    make_vocab_size_divisible_by: int = 1

    def __post_init__(self):
        if self.num_kv_heads is None:
            self.num_kv_heads = self.num_heads

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads

    @property
    def padded_vocab_size(self) -> int:
        m = self.make_vocab_size_divisible_by
        return (self.vocab_size + m - 1) // m * m


@dataclass
class LayerStrategy:
    """Parallel layout of one module. ``tp`` is the width of the tensor/sequence-parallel group; ``sp`` says what
    it does: "none" (Megatron TP, activations replicated), "megatron" (TP + sequence parallel) or "ulysses"
    (full weights, sequence-sharded activations, head-sharded attention)."""
    tp: int = 1
    sp: str = "none"
    cp: int = 1
    dp_type: str = "ddp"
    checkpoint: bool = False
    tp_group: Any = None      # CommGroup of size tp
    cp_group: Any = None
    wdp_group: Any = None     # weight-replica group (gradient reduction / ZeRO sharding)
    impl: str = "nccl"        # nccl | fused
    tp_rank: int = 0
    cp_rank: int = 0

    @property
    def weight_tp(self) -> int:
        return 1 if self.sp == "ulysses" else self.tp

    @property
    def seq_shards(self) -> int:
        """How many ways the sequence dimension of the block's input/output is split."""
        return (self.tp if self.sp in ("megatron", "ulysses") else 1) * self.cp

    def pg(self):
        return self.tp_group.group if self.tp_group is not None else None

    def linear_cfg(self, kind: str) -> A.LinearCfg:
        if self.weight_tp == 1:
            return A.LinearCfg("plain", None, self.impl)
        mode = kind + ("_sp" if self.sp == "megatron" else "")
        return A.LinearCfg(mode, self.pg(), self.impl)


_FULL_SEQUENCE = LayerStrategy()       # layout of an activation that holds the whole sequence (before any scatter)


@dataclass
class BatchCtx:
    """Per-micro-batch metadata that travels with the activations through a stage."""
    batch: int                      # local micro-batch size under the current layout
    seq: int                        # full sequence length
    labels: Optional[torch.Tensor] = None       # [seq(_local), batch] token labels or [batch] class labels
    loss_mask: Optional[torch.Tensor] = None
    positions: Optional[torch.Tensor] = None    # explicit per-token positions (context parallel zigzag)
    extra: dict = field(default_factory=dict)


def hidden_dropout(x: torch.Tensor, p: float, ctx: "BatchCtx", st: "LayerStrategy", site: int) -> torch.Tensor:
    """Inverted dropout on a sequence-major activation [rows_local, h] (hidden / embedding dropout of GPT, BERT, ViT, T5;
    the reference draws these masks under a forked CUDA RNG tracker, models/gpt_hf/GPTModel_sequential.py:91-95).

    The mask is a pure function of (seed, iteration, micro-batch, data-parallel position, site): a counter-based draw,
    so the recomputed forward of a checkpointed block sees the same mask without saving RNG state, replicated
    activations get identical masks on every tensor-parallel rank, and a sequence-sharded activation takes its rows of
    the mask of the whole sequence (the same elements are dropped under TP = 1, TP and TP + sequence parallelism)."""
    key = ctx.extra.get("rng")
    if p <= 0.0 or key is None:
        return x
    parts = st.seq_shards
    idx = st.cp_rank * (st.tp if st.sp in ("megatron", "ulysses") else 1) + (st.tp_rank if st.sp in ("megatron", "ulysses") else 0)
    seed = 0x9E3779B97F4A7C15
    for v in (*key, site):
        seed = ((seed ^ (int(v) + 0x7F4A7C15)) * 0x100000001B3) % (1 << 63)
    g = torch.Generator(device=x.device)
    g.manual_seed(seed)
    rows = x.shape[0]
    mask = torch.empty(rows * parts, x.shape[1], dtype=x.dtype, device=x.device).bernoulli_(1.0 - p, generator=g)
    if parts > 1:
        mask = mask[idx * rows:(idx + 1) * rows]
    return x * mask * (1.0 / (1.0 - p))


_DEFER_INIT = {"on": False}


class deferred_init:
    """Build modules without initial values (reference: ``init_empty_weights`` + FSDP ``param_init_fn`` that loads a
    checkpoint while materialising, galvatron/core/runtime/initialize.py:7-104, parallel.py:79-89). Inside this context
    a weight gets its storage but no values: the (host-side, seeded) random generation of every full tensor -- most of
    the construction time of a large model -- is skipped. Use it when every weight is about to be read from a
    checkpoint (``--initialize_on_meta 1`` with ``--load``)."""

    def __enter__(self):
        self.prev = _DEFER_INIT["on"]
        _DEFER_INIT["on"] = True
        return self

    def __exit__(self, *exc):
        _DEFER_INIT["on"] = self.prev
        return False


def _det_normal(shape, std, seed, device, dtype):
    """Deterministic normal init independent of the device and of how the tensor is later sharded."""
    if _DEFER_INIT["on"]:
        return torch.empty(shape, device=device, dtype=dtype)      # storage only: the loader fills it
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    if math.prod(shape) > (1 << 24) and str(device) != "cpu":
        gd = torch.Generator(device=device)
        gd.manual_seed(seed)
        return (torch.randn(shape, generator=gd, device=device, dtype=torch.float32) * std).to(dtype)
    return (torch.randn(shape, generator=g, dtype=torch.float32) * std).to(device=device, dtype=dtype)


def _shard_rows(w: torch.Tensor, parts: int, idx: int) -> torch.Tensor:
    n = w.shape[0] // parts
    return w[idx * n:(idx + 1) * n].contiguous()


def _shard_cols(w: torch.Tensor, parts: int, idx: int) -> torch.Tensor:
    n = w.shape[1] // parts
    return w[:, idx * n:(idx + 1) * n].contiguous()


class Norm(nn.Module):
    def __init__(self, cfg: ModelConfig, device, sequence_parallel: bool, tp_duplicate: bool):
        super().__init__()
        self.kind, self.eps = cfg.norm, cfg.norm_eps
        self.weight = nn.Parameter(torch.ones(cfg.hidden_size, dtype=cfg.dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(cfg.hidden_size, dtype=cfg.dtype, device=device)) if cfg.norm == "layer" else None
        for p in self.parameters():
            p.sequence_parallel = sequence_parallel
            p.tp_duplicate = tp_duplicate

    def forward(self, x):
        if self.kind == "rms":
            return A.rmsnorm(x, self.weight, self.eps)
        return A.layernorm(x, self.weight, self.bias, self.eps)

    def branch(self, x):
        """(norm(x), x): the pre-norm branch point; use the second value as the residual so that its gradient is added
        inside the norm's backward kernel."""
        if self.kind == "rms":
            return A.rmsnorm_branch(x, self.weight, self.eps)
        return A.layernorm_branch(x, self.weight, self.bias, self.eps)


def attention_dropout_spec(cfg: "ModelConfig", ctx: "BatchCtx", layer_idx: int, head_offset: int, cross: bool = False):
    """(p, seed, head offset) for the attention kernels, or None when no dropout applies to this call. The seed folds the
    step's dropout key (seed, iteration, micro-batch, data-parallel position) and the layer, the kernels fold batch
    element, GLOBAL head index and (query, key) position, so the mask does not depend on how heads are split over
    tensor-parallel ranks and repeats in a recomputed forward (reference: attention dropout under the forked CUDA RNG
    tracker, galvatron/core/runtime/tensor_parallel/transformer.py:353,397,451-479)."""
    key = ctx.extra.get("rng")
    p = cfg.dropout if cfg.attention_dropout is None else cfg.attention_dropout
    if key is None or p <= 0.0:
        return None
    seed = 0x51ED270B7F4A7C15
    for v in (*key, 2 * layer_idx + int(cross)):
        seed = ((seed ^ (int(v) + 0x9E3779B9)) * 0x100000001B3) % (1 << 63)
    return (float(p), seed, int(head_offset))


def key_lengths(ctx: "BatchCtx", name: str = "attention_mask"):
    """Per-sequence count of real keys from a padding mask [batch, seq] in the batch's extras (1 = token, 0 = padding,
    padding on the right, as HuggingFace tokenizers produce it); None when the batch carries no such mask. The reference
    feeds these masks to its attention modules (galvatron/models/bert_hf/BertModel_sequential.py:12-15,
    galvatron/models/T5/T5Model_tensor_parallel.py:96-115); here they reach the attention kernel as key lengths."""
    mask = ctx.extra.get(name)
    if mask is None:
        return None
    key = "_lens_" + name
    lens = ctx.extra.get(key)
    if lens is None:
        if mask.shape[0] != ctx.batch:
            raise ValueError("padding mask for %d sequences, layer runs %d: padding masks need a layout that keeps the "
                             "micro-batch of the data layout" % (mask.shape[0], ctx.batch))
        lens = mask.to(torch.int32).sum(dim=1).to(torch.int32)
        ctx.extra[key] = lens
    return lens


def relative_position_buckets(sq: int, sk: int, bidirectional: bool, num_buckets: int, max_distance: int) -> torch.Tensor:
    """[sq, sk] bucket index of the offset (key position - query position), as defined for T5 (Raffel et al. 2020, section
    2.1): half of the buckets for each direction when ``bidirectional`` (else future keys all fall into bucket 0), the first
    half of a direction's buckets for exact small offsets, the rest spaced logarithmically up to ``max_distance``, beyond
    which every offset shares the last bucket."""
    rel = torch.arange(sk)[None, :] - torch.arange(sq)[:, None]
    out = torch.zeros_like(rel)
    n = num_buckets
    if bidirectional:
        n //= 2
        out = out + (rel > 0).long() * n
        dist = rel.abs()
    else:
        dist = (-rel).clamp(min=0)
    exact = n // 2
    far = exact + (torch.log(dist.clamp(min=1).float() / exact) / math.log(max_distance / exact) * (n - exact)).long()
    return out + torch.where(dist < exact, dist, far.clamp(max=n - 1))


class SelfAttention(nn.Module):
    """Fused QKV projection -> (RoPE) -> flash attention -> output projection (+ residual)."""

    def __init__(self, cfg: ModelConfig, st: LayerStrategy, layer_idx: int, device, cross: bool = False):
        super().__init__()
        self.cfg, self.st, self.cross, self.layer_idx = cfg, st, cross, layer_idx
        h, dh = cfg.hidden_size, cfg.head_dim
        t, r = st.weight_tp, st.tp_rank if st.weight_tp > 1 else 0
        assert cfg.num_heads % st.tp == 0, "heads must divide by the tensor/sequence-parallel degree"
        hq, hk = cfg.num_heads, cfg.num_kv_heads
        assert hk % t == 0, "tensor parallelism needs the KV-head count divisible by the tp degree"
        self.hq_w, self.hk_w = hq // t, hk // t             # heads held in the weights of this rank
        seed = 1000 + layer_idx * 16 + (8 if cross else 0)
        wq = _det_normal((hq * dh, h), cfg.init_std, seed + 1, device, cfg.dtype)
        wk = _det_normal((hk * dh, h), cfg.init_std, seed + 2, device, cfg.dtype)
        wv = _det_normal((hk * dh, h), cfg.init_std, seed + 3, device, cfg.dtype)
        wo = _det_normal((h, hq * dh), cfg.init_std / math.sqrt(2.0 * max(cfg.num_layers, 1)), seed + 4, device, cfg.dtype)
        self.wqkv = nn.Parameter(torch.cat([_shard_rows(wq, t, r), _shard_rows(wk, t, r), _shard_rows(wv, t, r)], 0))
        self.wo = nn.Parameter(_shard_cols(wo, t, r))
        if cfg.bias:
            self.bqkv = nn.Parameter(torch.zeros(self.wqkv.shape[0], dtype=cfg.dtype, device=device))
            self.bo = nn.Parameter(torch.zeros(h, dtype=cfg.dtype, device=device))
            self.bo.tp_duplicate = t > 1
            self.bo.sequence_parallel = st.sp == "megatron" and t > 1
        else:
            self.bqkv = self.bo = None
        if cfg.pos == "rope":
            self.register_buffer("inv_freq", Fn.rope_inv_freq(dh, cfg.rope_base, device), persistent=False)
        else:
            self.inv_freq = None
        self.rel_bias = None
        if cfg.relative_attention_num_buckets > 0 and not cross:
            assert hq == hk, "relative position bias is defined for multi-head attention (as many key heads as query heads)"
            table = _det_normal((cfg.relative_attention_num_buckets, hq), cfg.init_std, seed + 5, device, cfg.dtype)
            self.rel_bias = nn.Parameter(table[:, r * self.hq_w:(r + 1) * self.hq_w].contiguous())     # this rank's heads
            self._bucket_cache: dict = {}

    def _position_bias(self, s: int, causal: bool, device) -> torch.Tensor:
        """[heads, s, s] additive score term: the table entry of every (query, key) offset, and for causal attention a
        large negative constant on future keys."""
        key = (s, causal, str(device))
        cached = self._bucket_cache.get(key)
        if cached is None:
            cfg = self.cfg
            idx = relative_position_buckets(s, s, not causal, cfg.relative_attention_num_buckets, cfg.relative_attention_max_distance)
            future = torch.zeros(s, s).masked_fill(torch.arange(s)[None, :] > torch.arange(s)[:, None], -30000.0) if causal else None
            cached = (idx.reshape(-1).to(device), None if future is None else future.to(device=device, dtype=cfg.dtype))
            self._bucket_cache[key] = cached
        idx, future = cached
        bias = self.rel_bias.index_select(0, idx).view(s, s, self.hq_w).permute(2, 0, 1)
        return bias if future is None else bias + future

    def _biased(self, qkv: torch.Tensor, ctx: BatchCtx, causal: bool, kv_lens) -> torch.Tensor:
        """Self-attention with the relative position bias: q / k / v as strided views of the packed projection, the bias
        (shared by the batch) and the padding mask (per sequence) as additive terms of ``A.biased_attention``. Dropout of the
        attention probabilities is not applied on this path (hidden dropout is, by the enclosing layer)."""
        b, dh, hq, hk = ctx.batch, self.cfg.head_dim, self.hq_w, self.hk_w
        s = qkv.shape[0] // b
        q = qkv[:, :hq * dh].reshape(s, b, hq, dh).transpose(0, 1)
        k = qkv[:, hq * dh:(hq + hk) * dh].reshape(s, b, hk, dh).transpose(0, 1)
        v = qkv[:, (hq + hk) * dh:].reshape(s, b, hk, dh).transpose(0, 1)
        mask = None
        if kv_lens is not None:
            padded = torch.arange(s, device=qkv.device)[None, :] >= kv_lens[:, None].to(qkv.device)            # [b, s] keys
            mask = torch.zeros(b, 1, s, dtype=torch.float32, device=qkv.device).masked_fill(padded[:, None, :], -30000.0)
            mask = mask.expand(b, s, s).contiguous()
        o = A.biased_attention(q, k, v, bias=self._position_bias(s, causal, qkv.device), mask=mask)
        return o.transpose(0, 1).reshape(s * b, hq * dh)

    def forward(self, x, residual, ctx: BatchCtx, kv_source=None, causal=None):
        cfg, st = self.cfg, self.st
        causal = cfg.causal if causal is None else causal
        rope = cfg.pos == "rope" and not self.cross
        if self.cross:
            return self._cross(x, residual, ctx, kv_source)
        kv_lens = key_lengths(ctx, "decoder_attention_mask" if getattr(self, "is_decoder", False) else "attention_mask")
        if kv_lens is not None and (st.cp > 1 or (st.sp == "ulysses" and st.tp > 1)):
            raise NotImplementedError("padding masks are supported with tensor / data / pipeline parallelism, not with "
                                      "sequence-sharded attention (Ulysses, context parallelism)")
        if self.rel_bias is not None and (st.cp > 1 or (st.sp == "ulysses" and st.tp > 1)):
            raise NotImplementedError("relative position bias is supported with tensor / Megatron sequence / data / pipeline "
                                      "parallelism, not with sequence-sharded attention (Ulysses, context parallelism)")
        if (st.sp == "ulysses" and st.tp > 1 and st.impl == "fused" and x.is_cuda and x.dtype == torch.bfloat16
                and cfg.num_kv_heads >= st.tp and st.cp == 1):
            from ..parallel.ulysses import ulysses_block_fused
            return ulysses_block_fused(x, residual, self, ctx, causal, rope)
        lcfg = st.linear_cfg("col")
        # RoPE in the projection's epilogue when the projection is a plain GEMM whose rows are whole-sequence tokens
        fuse_rope = (rope and st.cp == 1 and not (st.sp == "ulysses" and st.tp > 1) and ctx.positions is None
                     and not (lcfg.mode == "col_sp" and lcfg.impl == "fused") and RopeEpilogue.supported(x, cfg.head_dim, self.bqkv))
        rope_ep = RopeEpilogue((self.hq_w + self.hk_w) * cfg.head_dim, cfg.head_dim, self.inv_freq, None, ctx.batch, 0) if fuse_rope else None
        qkv = A.linear(x, self.wqkv, self.bqkv, None, lcfg, rope=rope_ep)
        if self.rel_bias is not None:
            return A.linear(self._biased(qkv, ctx, causal, kv_lens), self.wo, self.bo, residual, st.linear_cfg("row"))
        if st.sp == "ulysses" and st.tp > 1:
            from ..parallel.ulysses import ulysses_attention
            o = ulysses_attention(qkv, self, ctx, causal, rope)
        elif st.cp > 1:
            from ..parallel.ring_attention import ring_attention_packed
            o = ring_attention_packed(qkv, self, ctx, causal, rope)
        else:
            s_off = 0
            drop = attention_dropout_spec(cfg, ctx, self.layer_idx, (st.tp_rank if st.weight_tp > 1 else 0) * self.hq_w)
            acfg = A.AttnCfg(batch=ctx.batch, hq=self.hq_w, hk=self.hk_w, dh=cfg.head_dim, causal=causal, rope=rope,
                             pos_offset=s_off, rope_applied=fuse_rope, dropout=drop)
            o = A.packed_attention(qkv, acfg, self.inv_freq, ctx.positions if rope else None, kv_lens)
        return A.linear(o, self.wo, self.bo, residual, st.linear_cfg("row"))

    def _cross(self, x, residual, ctx, kv_source):
        cfg, st = self.cfg, self.st
        dh = cfg.head_dim
        nq = self.hq_w * dh
        q = A.linear(x, self.wqkv[:nq], None if self.bqkv is None else self.bqkv[:nq], None, st.linear_cfg("col"))
        kv = A.linear(kv_source, self.wqkv[nq:], None if self.bqkv is None else self.bqkv[nq:], None, st.linear_cfg("col"))
        b = ctx.batch
        sq, sk = q.shape[0] // b, kv.shape[0] // b
        qv = q.view(sq, b, self.hq_w, dh).transpose(0, 1)
        kk = kv[:, : self.hk_w * dh].reshape(sk, b, self.hk_w, dh).transpose(0, 1)
        vv = kv[:, self.hk_w * dh:].reshape(sk, b, self.hk_w, dh).transpose(0, 1)
        drop = attention_dropout_spec(cfg, ctx, self.layer_idx, (st.tp_rank if st.weight_tp > 1 else 0) * self.hq_w, cross=True)
        o, _ = A.attention(qv, kk, vv, False, None, key_lengths(ctx, "attention_mask"), drop)    # keys = encoder tokens
        o = o.transpose(0, 1).reshape(sq * b, nq)
        return A.linear(o, self.wo, self.bo, residual, st.linear_cfg("row"))


class MLP(nn.Module):
    def __init__(self, cfg: ModelConfig, st: LayerStrategy, layer_idx: int, device):
        super().__init__()
        self.cfg, self.st = cfg, st
        h, f = cfg.hidden_size, cfg.ffn_hidden_size
        t, r = st.weight_tp, st.tp_rank if st.weight_tp > 1 else 0
        seed = 5000 + layer_idx * 16
        if cfg.act == "swiglu":
            wg = _det_normal((f, h), cfg.init_std, seed + 1, device, cfg.dtype)
            wu = _det_normal((f, h), cfg.init_std, seed + 2, device, cfg.dtype)
            self.w_up = nn.Parameter(torch.cat([_shard_rows(wg, t, r), _shard_rows(wu, t, r)], 0))
        else:
            wu = _det_normal((f, h), cfg.init_std, seed + 1, device, cfg.dtype)
            self.w_up = nn.Parameter(_shard_rows(wu, t, r))
        wd = _det_normal((h, f), cfg.init_std / math.sqrt(2.0 * max(cfg.num_layers, 1)), seed + 3, device, cfg.dtype)
        self.w_down = nn.Parameter(_shard_cols(wd, t, r))
        if cfg.bias:
            self.b_up = nn.Parameter(torch.zeros(self.w_up.shape[0], dtype=cfg.dtype, device=device))
            self.b_down = nn.Parameter(torch.zeros(h, dtype=cfg.dtype, device=device))
            self.b_down.tp_duplicate = t > 1
            self.b_down.sequence_parallel = st.sp == "megatron" and t > 1
        else:
            self.b_up = self.b_down = None

    def forward(self, x, residual):
        st = self.st
        if (self.cfg.act == "swiglu" and st.weight_tp == 1 and self.b_up is None and A.SAVE_SWIGLU_ACT
                and A.swiglu_epilogue_supported(x, self.w_up)):
            return A.swiglu_mlp(x, self.w_up, self.w_down, residual)     # activation in the up-projection's epilogue
        up = A.linear(x, self.w_up, self.b_up, None, st.linear_cfg("col"))
        if self.cfg.act == "swiglu":
            return A.swiglu_linear(up, self.w_down, residual, st.linear_cfg("row"))
        act = torch.relu(up) if self.cfg.act == "relu" else A.gelu(up)          # relu: the original T5 feed-forward
        return A.linear(act, self.w_down, self.b_down, residual, st.linear_cfg("row"))


class TransformerLayer(nn.Module):
    """Pre-LN (GPT / Llama / ViT / T5) or post-LN (BERT) block; optional cross-attention (T5 decoder)."""

    def __init__(self, cfg: ModelConfig, st: LayerStrategy, layer_idx: int, device, cross_attention: bool = False,
                 causal: Optional[bool] = None):
        super().__init__()
        self.cfg, self.st, self.causal, self.layer_idx = cfg, st, causal, layer_idx
        sp = st.sp == "megatron" and st.tp > 1
        dup = st.weight_tp > 1
        self.ln1 = Norm(cfg, device, sp, dup)
        self.attn = SelfAttention(cfg, st, layer_idx, device)
        self.ln2 = Norm(cfg, device, sp, dup)
        self.mlp = MLP(cfg, st, layer_idx, device)
        if cross_attention:
            self.ln_x = Norm(cfg, device, sp, dup)
            self.xattn = SelfAttention(cfg, st, layer_idx, device, cross=True)
            self.attn.is_decoder = True           # its padding mask is the decoder's, not the encoder's
        else:
            self.xattn = None

    def forward(self, h, ctx: BatchCtx, enc=None):
        p = self.cfg.dropout if ctx.extra.get("rng") is not None else 0.0
        if p > 0.0:
            return self._forward_with_dropout(h, ctx, enc, p)
        if self.cfg.post_ln:
            h = self.ln1(self.attn(h, h, ctx, causal=self.causal))
            return self.ln2(self.mlp(h, h))
        y, h = self.ln1.branch(h)
        h = self.attn(y, h, ctx, causal=self.causal)
        if self.xattn is not None:
            y, h = self.ln_x.branch(h)
            h = self.xattn(y, h, ctx, kv_source=enc)
        y, h = self.ln2.branch(h)
        return self.mlp(y, h)

    def _forward_with_dropout(self, h, ctx: BatchCtx, enc, p: float):
        """Same block with dropout on every sub-layer output before its residual add (the residual is then added
        here instead of in the projection's epilogue)."""
        st, base = self.st, 16 * (self.layer_idx + 1)
        drop = lambda y, site: hidden_dropout(y, p, ctx, st, base + site)
        if self.cfg.post_ln:
            h = self.ln1(h + drop(self.attn(h, None, ctx, causal=self.causal), 0))
            return self.ln2(h + drop(self.mlp(h, None), 1))
        h = h + drop(self.attn(self.ln1(h), None, ctx, causal=self.causal), 0)
        if self.xattn is not None:
            h = h + drop(self.xattn(self.ln_x(h), None, ctx, kv_source=enc), 2)
        return h + drop(self.mlp(self.ln2(h), None), 1)


def _local_seq_slice(x2: torch.Tensor, batch: int, parts: int, idx: int) -> torch.Tensor:
    """Rows of sequence chunk ``idx`` (of ``parts``) of a sequence-major [s * b, h] tensor."""
    if parts == 1:
        return x2
    rows = x2.shape[0] // parts
    return x2[idx * rows:(idx + 1) * rows]


class TokenEmbedding(nn.Module):
    """Vocab-parallel token embedding (+ learned positions, + token types); output in the layout of ``st``:
    sequence-sharded when ``st`` is sequence parallel (reference: LlamaModel_sequential.py:44-67)."""

    def __init__(self, cfg: ModelConfig, st: LayerStrategy, device, seed: int = 11):
        super().__init__()
        self.cfg, self.st = cfg, st
        t, r = st.weight_tp, st.tp_rank if st.weight_tp > 1 else 0
        V = cfg.padded_vocab_size
        assert V % t == 0, "vocab size must divide by the vocab tensor-parallel degree"
        full = _det_normal((V, cfg.hidden_size), cfg.init_std, seed, device, cfg.dtype)
        self.vocab_start = r * (V // t)
        self.wte = nn.Parameter(_shard_rows(full, t, r))
        self.wte.tied = cfg.tie_embeddings
        if cfg.pos == "learned":
            self.wpe = nn.Parameter(_det_normal((cfg.seq_length, cfg.hidden_size), cfg.init_std, seed + 1, device, cfg.dtype))
            self.wpe.tp_duplicate = t > 1
        else:
            self.wpe = None
        if cfg.type_vocab_size:
            self.wtt = nn.Parameter(_det_normal((cfg.type_vocab_size, cfg.hidden_size), cfg.init_std, seed + 2, device, cfg.dtype))
            self.wtt.tp_duplicate = t > 1
            self.ln = Norm(cfg, device, False, t > 1)
        else:
            self.wtt = None
            self.ln = None

    def forward(self, ids: torch.Tensor, ctx: BatchCtx):
        """ids: [s_in, b] where s_in is the full sequence (TP layouts) or this rank's slice (Ulysses / CP)."""
        st = self.st
        s_in, b = ids.shape
        pos_ids = None
        if self.wpe is not None:
            if ctx.positions is not None:
                pos_ids = ctx.positions.view(s_in, 1).expand(s_in, b)
            else:
                off = ctx.extra.get("seq_offset", 0)
                pos_ids = (torch.arange(s_in, device=ids.device) + off).view(s_in, 1).expand(s_in, b)
        t = st.weight_tp
        if t > 1:
            h = A.embedding(ids, self.wte, None, None, self.vocab_start, st.pg())
            if self.wpe is not None:
                h = h + A.embedding(pos_ids, self.wpe)
        else:
            h = A.embedding(ids, self.wte, pos_ids, self.wpe, 0, None)
        h = h.view(s_in * b, self.cfg.hidden_size)
        if self.wtt is not None:
            tt = ctx.extra.get("token_type_ids")
            if tt is not None:
                h = h + A.embedding(tt, self.wtt).view(s_in * b, -1)
            else:                                   # no segment ids: every token is segment 0
                h = h + self.wtt[0]
            h = self.ln(h)
        if self.cfg.dropout > 0.0 and ctx.extra.get("rng") is not None:
            h = hidden_dropout(h, self.cfg.dropout, ctx, _FULL_SEQUENCE if st.cp == 1 and st.sp != "ulysses" else st, 1)
        if st.sp == "megatron" and st.tp > 1:
            h = _ScatterSeq.apply(h, st.tp, st.tp_rank, st.pg())
        return h


class _ScatterSeq(torch.autograd.Function):
    """Keep this rank's sequence chunk; backward all-gathers (megatron mappings_group.py:192-206)."""

    @staticmethod
    def forward(ctx, x, parts, idx, group):
        ctx.group = group
        rows = x.shape[0] // parts
        return x[idx * rows:(idx + 1) * rows].contiguous()

    @staticmethod
    def backward(ctx, dy):
        return C.all_gather_first_dim(dy.contiguous(), ctx.group), None, None, None


class _GatherSeq(torch.autograd.Function):
    """All-gather sequence chunks; backward keeps this rank's chunk of the gradient."""

    @staticmethod
    def forward(ctx, x, parts, idx, group):
        ctx.parts, ctx.idx = parts, idx
        return C.all_gather_first_dim(x.contiguous(), group)

    @staticmethod
    def backward(ctx, dy):
        rows = dy.shape[0] // ctx.parts
        return dy[ctx.idx * rows:(ctx.idx + 1) * rows].contiguous(), None, None, None


class FinalNorm(nn.Module):
    def __init__(self, cfg: ModelConfig, st: LayerStrategy, device):
        super().__init__()
        self.norm = Norm(cfg, device, st.sp == "megatron" and st.tp > 1, st.weight_tp > 1)

    def forward(self, h, ctx: BatchCtx):
        return self.norm(h)


class LMHead(nn.Module):
    """Vocab-parallel LM head + cross entropy; returns the mean loss over this rank's tokens."""

    def __init__(self, cfg: ModelConfig, st: LayerStrategy, device, seed: int = 13, tied: Optional[nn.Parameter] = None,
                 fp32_logits: bool = False):
        super().__init__()
        self.cfg, self.st, self.fp32_logits = cfg, st, fp32_logits
        t, r = st.weight_tp, st.tp_rank if st.weight_tp > 1 else 0
        V = cfg.padded_vocab_size
        self.vocab_start = r * (V // t)
        if tied is not None:
            self.weight = tied
        else:
            full = _det_normal((V, cfg.hidden_size), cfg.init_std, 11 if cfg.tie_embeddings else seed, device, cfg.dtype)
            self.weight = nn.Parameter(_shard_rows(full, t, r))
            self.weight.tied = cfg.tie_embeddings

    def forward(self, h, ctx: BatchCtx):
        st = self.st
        labels = ctx.labels
        mode = "col_sp" if (st.sp == "megatron" and st.tp > 1) else "col"
        lcfg = A.LossCfg(vocab_start=self.vocab_start, group=st.pg() if st.weight_tp > 1 else None,
                         ignore_index=-100, mode=mode, fp32_logits=self.fp32_logits)
        loss = A.lm_head_loss(h, self.weight, labels.reshape(-1), lcfg)
        if ctx.loss_mask is not None:
            m = ctx.loss_mask.reshape(-1).to(loss.dtype)
            return (loss * m).sum() / m.sum().clamp(min=1.0)
        valid = (labels.reshape(-1) != -100).sum().clamp(min=1)
        return loss.sum() / valid
