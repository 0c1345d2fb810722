"""Autograd Functions of the runtime, built on the kernels of ``ops.functional`` / ``ops.gemm``.

Weight gradients follow the "main_grad" protocol of Megatron's gradient-accumulation fusion
(reference: megatron/core/tensor_parallel/layers.py:498-509): when a parameter carries a
``main_grad`` buffer (a view into the flat gradient bucket owned by the ZeRO engine), the
weight-gradient GEMM accumulates straight into it and autograd sees ``None``; otherwise the
gradient is returned to autograd as usual.

Tensor-parallel communication is part of the linear Functions (``mode``):

=========  ==========================================  =========================================
mode       forward                                     backward
=========  ==========================================  =========================================
plain      y = x W^T                                    dx = dy W
col        y = x W_shard^T (x replicated)               dx = all_reduce(dy W_shard)
col_sp     y = all_gather_seq(x) W_shard^T              dx = reduce_scatter_seq(dy W_shard)
row        y = all_reduce(x_shard W_shard^T)            dx = dy W_shard
row_sp     y = reduce_scatter_seq(x_shard W_shard^T)    dx = all_gather_seq(dy) W_shard
=========  ==========================================  =========================================
(reference: layers.py:399-417,435-494 column-parallel, :1092-1114 row-parallel.)
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import Any, Optional

import torch

from ..parallel import collectives as C
from . import functional as Fn
from .gemm import gemm, head_xent_grad, head_xent_stats, head_xent_supported, swiglu_epilogue_supported


# --------------------------------------------------------------------------- helpers
def _accum_param_grad(param: torch.Tensor, compute_into, compute_fresh):
    """Accumulate into ``param.main_grad`` when present (returns None), else return a fresh gradient."""
    mg = getattr(param, "main_grad", None)
    if mg is not None:
        compute_into(mg)
        hook = getattr(param, "grad_ready_hook", None)
        if hook is not None:
            hook(param)
        return None
    return compute_fresh()


def _wgrad(W: torch.Tensor, dy2: torch.Tensor, x2: torch.Tensor):
    return _accum_param_grad(
        W,
        lambda mg: gemm(dy2, x2, a_mn=True, b_mn=True, out=mg.view(W.shape), accumulate=True),
        lambda: gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=W.dtype))


def _vec_grad(p: torch.Tensor, fill_accum):
    """Gradient of a vector parameter (norm weight, bias): ``fill_accum(buf_fp32)`` adds into an fp32 buffer."""
    def into(mg):
        if mg.dtype == torch.float32:
            fill_accum(mg.view(-1))
        else:
            tmp = torch.zeros(p.numel(), dtype=torch.float32, device=p.device)
            fill_accum(tmp)
            mg.view(-1).add_(tmp.to(mg.dtype))

    def fresh():
        tmp = torch.zeros(p.numel(), dtype=torch.float32, device=p.device)
        fill_accum(tmp)
        return tmp.to(p.dtype).view(p.shape)

    return _accum_param_grad(p, into, fresh)


@dataclass(frozen=True)
class LinearCfg:
    mode: str = "plain"          # plain | col | col_sp | row | row_sp
    group: Any = None            # tensor-parallel process group
    impl: str = "nccl"           # "nccl" (library collective) or "fused" (peer-memory kernels)


# --------------------------------------------------------------------------- linear
class LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, W, bias, residual, cfg: LinearCfg, rope=None):
        n = C.group_size(cfg.group)
        mode = cfg.mode if n > 1 else "plain"
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        ctx.cfg, ctx.mode, ctx.lead = cfg, mode, lead
        ctx.has_bias, ctx.has_res = bias is not None, residual is not None
        if mode in ("row", "row_sp"):
            if cfg.impl == "fused" and x2.is_cuda:
                from ..parallel import fused
                y = fused.gemm_reduce(x2, W, cfg.group, scatter=(mode == "row_sp"), residual=residual, bias=bias)
            else:
                y = gemm(x2, W)
                y = C.all_reduce_(y, cfg.group) if mode == "row" else C.reduce_scatter_first_dim(y, cfg.group)
                if bias is not None:
                    y = y + bias
                if residual is not None:
                    y = y + residual.reshape(y.shape)
            out_lead = lead if mode == "row" else (lead[0] // n,) + tuple(lead[1:])
        else:
            if mode == "col_sp":
                if cfg.impl == "fused" and x2.is_cuda:
                    from ..parallel import fused
                    y = fused.allgather_gemm(x2, W, cfg.group, bias=bias)
                else:
                    xg = C.all_gather_first_dim(x2, cfg.group)
                    y = gemm(xg, W, bias=bias, rope=rope)
                out_lead = (lead[0] * n,) + tuple(lead[1:])
            else:
                y = gemm(x2, W, bias=bias, residual=None if residual is None else residual.reshape(-1, W.shape[0]), rope=rope)
                out_lead = lead
        ctx.save_for_backward(x2, W, bias)
        tgt = tuple(out_lead) + (W.shape[0],)
        return y if tuple(y.shape) == tgt else y.view(tgt)

    @staticmethod
    def backward(ctx, dy):
        x2, W, bias = ctx.saved_tensors
        cfg, mode = ctx.cfg, ctx.mode
        dy2 = dy.reshape(-1, W.shape[0])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dres = dy if ctx.has_res else None
        use_fused = cfg.impl == "fused" and dy2.is_cuda
        dx = None
        dyg = dy2
        if mode == "row_sp":
            if use_fused and ctx.needs_input_grad[0] and dy2.shape[0] % 128 == 0:
                from ..parallel import fused
                # all-gather(dy) -> dgrad GEMM in one kernel; the gathered dy comes back for the weight gradient
                dx, dyg = fused.allgather_gemm(dy2, W, cfg.group, return_gathered=True, b_mn=True)
                dx = dx.view(*ctx.lead, W.shape[1])
            else:
                dyg = C.all_gather_first_dim(dy2, cfg.group)
        if mode == "col_sp":
            if use_fused:
                from ..parallel import fused
                xg = fused.allgather_pull(x2, fused.comm_group(cfg.group), "xg").view(-1, x2.shape[1])
            else:
                xg = C.all_gather_first_dim(x2, cfg.group)
        else:
            xg = x2
        if ctx.needs_input_grad[0] and dx is None:
            if mode == "col_sp" and use_fused:
                from ..parallel import fused
                dx = fused.gemm_reduce(dyg, W, cfg.group, scatter=True, b_mn=True)   # dgrad GEMM -> reduce-scatter
            else:
                dx = gemm(dyg, W, b_mn=True)
                if mode == "col":
                    C.all_reduce_(dx, cfg.group)
                elif mode == "col_sp":
                    dx = C.reduce_scatter_first_dim(dx, cfg.group)
            dx = dx.view(*ctx.lead, W.shape[1])
        dW = _wgrad(W, dyg, xg)
        db = None
        if ctx.has_bias:
            db = _vec_grad(bias, lambda buf: Fn.colsum_accum(dy2 if mode in ("row", "row_sp") else dyg, buf))
        return dx, dW, db, dres, None, None


def linear(x, W, bias=None, residual=None, cfg: LinearCfg = LinearCfg(), rope=None):
    """``rope`` (a ``gemm.RopeEpilogue``): the projection's epilogue rotates its q / k head columns. This Function's
    backward treats the rotated output as its output, so the consumer's backward must hand back the gradient with the
    inverse rotation applied (``PackedAttentionFn`` does, for ``AttnCfg.rope`` with ``rope_applied``)."""
    return LinearFn.apply(x, W, bias, residual, cfg, rope)


# Keep silu(gate) * up for the backward pass (one [tokens, ffn] bf16 tensor per layer) instead of recomputing it
# from the gate / up projection there. GV_SAVE_SWIGLU_ACT=0 trades the extra pass back for the memory.
SAVE_SWIGLU_ACT = os.environ.get("GV_SAVE_SWIGLU_ACT", "1") != "0"


class SwiGLULinearFn(torch.autograd.Function):
    """y = (silu(gate) * up) W^T (+ residual); the activation is saved for the weight-gradient GEMM (or recomputed in
    backward when ``SAVE_SWIGLU_ACT`` is off)."""

    @staticmethod
    def forward(ctx, gu, W, residual, cfg: LinearCfg):
        n = C.group_size(cfg.group)
        mode = cfg.mode if n > 1 else "plain"
        lead = gu.shape[:-1]
        gu2 = gu.reshape(-1, gu.shape[-1])
        a = Fn.swiglu_fwd(gu2)
        ctx.cfg, ctx.mode, ctx.lead, ctx.has_res = cfg, mode, lead, residual is not None
        if mode in ("row", "row_sp"):
            if cfg.impl == "fused" and a.is_cuda:
                from ..parallel import fused
                y = fused.gemm_reduce(a, W, cfg.group, scatter=(mode == "row_sp"), residual=residual)
            else:
                y = gemm(a, W)
                y = C.all_reduce_(y, cfg.group) if mode == "row" else C.reduce_scatter_first_dim(y, cfg.group)
                if residual is not None:
                    y = y + residual.reshape(y.shape)
            out_lead = lead if mode == "row" else (lead[0] // n,) + tuple(lead[1:])
        else:
            y = gemm(a, W, residual=None if residual is None else residual.reshape(-1, W.shape[0]))
            out_lead = lead
        ctx.save_for_backward(gu2, W, a if SAVE_SWIGLU_ACT else None)
        tgt = tuple(out_lead) + (W.shape[0],)
        return y if tuple(y.shape) == tgt else y.view(tgt)

    @staticmethod
    def backward(ctx, dy):
        gu2, W, a = ctx.saved_tensors
        cfg, mode = ctx.cfg, ctx.mode
        dy2 = dy.reshape(-1, W.shape[0])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        if mode == "row_sp" and cfg.impl == "fused" and dy2.is_cuda and dy2.shape[0] % 128 == 0:
            from ..parallel import fused
            da, dyg = fused.allgather_gemm(dy2, W, cfg.group, return_gathered=True, b_mn=True)
        else:
            dyg = C.all_gather_first_dim(dy2, cfg.group) if mode == "row_sp" else dy2
            da = gemm(dyg, W, b_mn=True)
        if a is None:
            a = Fn.swiglu_fwd(gu2)
        dW = _wgrad(W, dyg, a)
        del a
        dgu = Fn.swiglu_bwd(da, gu2).view(*ctx.lead, gu2.shape[-1])
        return dgu, dW, (dy if ctx.has_res else None), None


def swiglu_linear(gu, W, residual=None, cfg: LinearCfg = LinearCfg()):
    return SwiGLULinearFn.apply(gu, W, residual, cfg)


class SwiGLUMLPFn(torch.autograd.Function):
    """Whole gated MLP of an un-sharded layer: y = (silu(x Wg^T) * (x Wu^T)) Wd^T + residual, with the activation
    computed in the up-projection's epilogue (no separate pass over the [tokens, 2 ffn] projection) and the residual
    added in the down-projection's epilogue. Saves the projection and the activation for the backward pass."""

    @staticmethod
    def forward(ctx, x, w_up, w_down, residual):
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        f = w_up.shape[0] // 2
        act = torch.empty(x2.shape[0], f, dtype=x2.dtype, device=x2.device)
        gu = gemm(x2, w_up, swiglu_out=act)
        y = gemm(act, w_down, residual=None if residual is None else residual.reshape(-1, w_down.shape[0]))
        ctx.lead, ctx.has_res = lead, residual is not None
        ctx.save_for_backward(x2, w_up, w_down, gu, act)
        return y.view(*lead, w_down.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w_up, w_down, gu, act = ctx.saved_tensors
        dy2 = dy.reshape(-1, w_down.shape[0])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        da = gemm(dy2, w_down, b_mn=True)
        dw_down = _wgrad(w_down, dy2, act)
        dgu = Fn.swiglu_bwd(da, gu)
        del da
        dx = gemm(dgu, w_up, b_mn=True).view(*ctx.lead, w_up.shape[1])
        dw_up = _wgrad(w_up, dgu, x2)
        return dx, dw_up, dw_down, (dy if ctx.has_res else None)


def swiglu_mlp(x, w_up, w_down, residual=None):
    return SwiGLUMLPFn.apply(x, w_up, w_down, residual)


class GeluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        ctx.save_for_backward(x)
        return Fn.gelu_fwd(x.contiguous())

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        return Fn.gelu_bwd(dy.contiguous(), x.contiguous())


def gelu(x):
    return GeluFn.apply(x)


# --------------------------------------------------------------------------- normalisation
class RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        y, _, rstd = Fn.rmsnorm_fwd(x, w, eps)
        ctx.save_for_backward(x, w, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, rstd = ctx.saved_tensors
        holder = {}

        def fill(buf):
            holder["dx"] = Fn.rmsnorm_bwd(dy, x, w, rstd, None, buf)

        dw = _vec_grad(w, fill)
        return holder["dx"], dw, None


def rmsnorm(x, w, eps: float = 1e-5):
    return RMSNormFn.apply(x, w, eps)


class RMSNormBranchFn(torch.autograd.Function):
    """Pre-norm branch point: returns (norm(x), x). The second output is the residual stream itself; routing it through
    this Function means the gradient of the residual branch arrives HERE, next to the gradient of the normalised
    branch, and the backward kernel adds it while it writes dx (``dres``) -- instead of autograd summing the two
    gradients of x with a separate element-wise kernel (the reference adds residuals with plain torch ops,
    galvatron/models/llama_hf/LlamaModel_tensor_parallel.py:81,96)."""

    @staticmethod
    def forward(ctx, x, w, eps):
        y, _, rstd = Fn.rmsnorm_fwd(x, w, eps)
        ctx.save_for_backward(x, w, rstd)
        return y, x.view_as(x)

    @staticmethod
    def backward(ctx, dy, dres):
        x, w, rstd = ctx.saved_tensors
        holder = {}
        if dy is None:
            return dres, None, None

        def fill(buf):
            holder["dx"] = Fn.rmsnorm_bwd(dy, x, w, rstd, dres, buf)

        dw = _vec_grad(w, fill)
        return holder["dx"], dw, None


def rmsnorm_branch(x, w, eps: float = 1e-5):
    return RMSNormBranchFn.apply(x, w, eps)


class LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, eps):
        y, _, mean, rstd = Fn.layernorm_fwd(x, w, b, eps)
        ctx.save_for_backward(x, w, b, mean, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, b, mean, rstd = ctx.saved_tensors
        dwb = torch.zeros(2, w.numel(), dtype=torch.float32, device=w.device)
        dx = Fn.layernorm_bwd(dy, x, w, mean, rstd, None, dwb[0], dwb[1])
        dw = _vec_grad(w, lambda buf: buf.add_(dwb[0]))
        db = _vec_grad(b, lambda buf: buf.add_(dwb[1]))
        return dx, dw, db, None


def layernorm(x, w, b, eps: float = 1e-5):
    return LayerNormFn.apply(x, w, b, eps)


class LayerNormBranchFn(torch.autograd.Function):
    """(layernorm(x), x) with the residual-branch gradient added inside the backward kernel; see ``RMSNormBranchFn``."""

    @staticmethod
    def forward(ctx, x, w, b, eps):
        y, _, mean, rstd = Fn.layernorm_fwd(x, w, b, eps)
        ctx.save_for_backward(x, w, b, mean, rstd)
        return y, x.view_as(x)

    @staticmethod
    def backward(ctx, dy, dres):
        x, w, b, mean, rstd = ctx.saved_tensors
        if dy is None:
            return dres, None, None, None
        dwb = torch.zeros(2, w.numel(), dtype=torch.float32, device=w.device)
        dx = Fn.layernorm_bwd(dy, x, w, mean, rstd, dres, dwb[0], dwb[1])
        dw = _vec_grad(w, lambda buf: buf.add_(dwb[0]))
        db = _vec_grad(b, lambda buf: buf.add_(dwb[1]))
        return dx, dw, db, None


def layernorm_branch(x, w, b, eps: float = 1e-5):
    return LayerNormBranchFn.apply(x, w, b, eps)


# --------------------------------------------------------------------------- attention
@dataclass(frozen=True)
class AttnCfg:
    """Packed-QKV attention over sequence-major tokens: qkv is [s * b, (hq + 2 hk) * dh]."""
    batch: int
    hq: int
    hk: int
    dh: int
    causal: bool = True
    rope: bool = False
    pos_offset: int = 0
    scale: Optional[float] = None
    rope_applied: bool = False      # the producer of qkv (a projection with a rotary epilogue) rotated q and k already
    dropout: Optional[tuple] = None   # (p, seed, head offset): dropout of the attention probabilities, counter-based


def _qkv_views(qkv: torch.Tensor, cfg: AttnCfg):
    tokens = qkv.shape[0]
    s = tokens // cfg.batch
    hq, hk, dh = cfg.hq, cfg.hk, cfg.dh
    q = qkv[:, : hq * dh].view(s, cfg.batch, hq, dh).transpose(0, 1)
    k = qkv[:, hq * dh:(hq + hk) * dh].view(s, cfg.batch, hk, dh).transpose(0, 1)
    v = qkv[:, (hq + hk) * dh:].view(s, cfg.batch, hk, dh).transpose(0, 1)
    return q, k, v


def _rope_packed_(qkv: torch.Tensor, cfg: AttnCfg, inv_freq, positions, inverse: bool):
    tokens = qkv.shape[0]
    hq, hk, dh = cfg.hq, cfg.hk, cfg.dh
    qv = qkv[:, : hq * dh].view(tokens, hq, dh)
    kv = qkv[:, hq * dh:(hq + hk) * dh].view(tokens, hk, dh)
    Fn.rope_(qv, inv_freq, cfg.batch, 0, cfg.pos_offset, positions, inverse)
    Fn.rope_(kv, inv_freq, cfg.batch, 0, cfg.pos_offset, positions, inverse)


class PackedAttentionFn(torch.autograd.Function):
    """RoPE (in place on the packed projection) + flash attention; output is [s * b, hq * dh]."""

    @staticmethod
    def forward(ctx, qkv, inv_freq, positions, cfg: AttnCfg, kv_lens=None):
        qkv = qkv if qkv.is_contiguous() else qkv.contiguous()
        if cfg.rope and not cfg.rope_applied:
            # in place on the projection output (detached: the rotation is part of this Function's math)
            _rope_packed_(qkv.detach(), cfg, inv_freq, positions, False)
        q, k, v = _qkv_views(qkv, cfg)
        tokens = qkv.shape[0]
        s = tokens // cfg.batch
        o = torch.empty(s, cfg.batch, cfg.hq, cfg.dh, dtype=qkv.dtype, device=qkv.device)
        _, lse = Fn.attention_fwd(q, k, v, cfg.causal, cfg.scale, out=o.transpose(0, 1), kv_lens=kv_lens, dropout=cfg.dropout)
        ctx.cfg = cfg
        ctx.save_for_backward(qkv, o, lse, inv_freq, positions, kv_lens)
        return o.view(tokens, cfg.hq * cfg.dh)

    @staticmethod
    def backward(ctx, dout):
        qkv, o, lse, inv_freq, positions, kv_lens = ctx.saved_tensors
        cfg = ctx.cfg
        tokens = qkv.shape[0]
        s = tokens // cfg.batch
        q, k, v = _qkv_views(qkv, cfg)
        dqkv = torch.empty_like(qkv)
        dq, dk, dv = _qkv_views(dqkv, cfg)
        do = dout.reshape(s, cfg.batch, cfg.hq, cfg.dh).transpose(0, 1)
        from . import attention as _attn
        # the native kernel's last stage (fp32 dq accumulator -> bf16) applies the inverse rotation of dq for free; the
        # key heads keep the separate in-place pass
        fold = cfg.rope and Fn._native(q) and _attn.supported(q, k, v) and cfg.dh % 16 == 0
        Fn.attention_bwd(do, q, k, v, o.transpose(0, 1), lse, cfg.causal, cfg.scale, dq, dk, dv, kv_lens=kv_lens,
                         dq_rope=(inv_freq, positions, cfg.pos_offset) if fold else None, dropout=cfg.dropout)
        if cfg.rope:
            if fold:
                kview = dqkv[:, cfg.hq * cfg.dh:(cfg.hq + cfg.hk) * cfg.dh].view(tokens, cfg.hk, cfg.dh)
                Fn.rope_(kview, inv_freq, cfg.batch, 0, cfg.pos_offset, positions, True)
            else:
                _rope_packed_(dqkv, cfg, inv_freq, positions, True)
        return dqkv, None, None, None, None


def packed_attention(qkv, cfg: AttnCfg, inv_freq=None, positions=None, kv_lens=None):
    """``kv_lens`` int [batch]: keys at or beyond kv_lens[b] are padding (the padding mask of encoder batches)."""
    return PackedAttentionFn.apply(qkv, inv_freq, positions, cfg, kv_lens)


class AttentionFn(torch.autograd.Function):
    """Flash attention over separate q [b, sq, hq, dh], k, v [b, sk, hk, dh] (any strides); returns (o, lse)."""

    @staticmethod
    def forward(ctx, q, k, v, causal, scale, kv_lens=None, dropout=None):
        o, lse = Fn.attention_fwd(q, k, v, causal, scale, kv_lens=kv_lens, dropout=dropout)
        ctx.causal, ctx.scale, ctx.dropout = causal, scale, dropout
        ctx.save_for_backward(q, k, v, o, lse, kv_lens)
        ctx.mark_non_differentiable(lse)
        return o, lse

    @staticmethod
    def backward(ctx, do, _dlse):
        q, k, v, o, lse, kv_lens = ctx.saved_tensors
        dq, dk, dv = Fn.attention_bwd(do, q, k, v, o, lse, ctx.causal, ctx.scale, kv_lens=kv_lens, dropout=ctx.dropout)
        return dq, dk, dv, None, None, None, None


def attention(q, k, v, causal: bool = True, scale: float | None = None, kv_lens=None, dropout=None):
    return AttentionFn.apply(q, k, v, causal, scale, kv_lens, dropout)


class BiasedAttentionFn(torch.autograd.Function):
    """Full (non-causal) attention with extra score terms on the tcgen05 kernels: q, k, v [b, s, h, dh] (any strides the
    kernels accept); ``bias`` [h, sq, sk] additive and shared by the batch (differentiable: its gradient is summed over
    the batch inside the backward kernel); ``mask`` [n, sq, sk] additive constant and ``ids`` [n, s] group ids (a query sees
    the keys of its own group) for batch element ``i % n``. Windowed attention of Swin: batch elements are windows, bias
    is the relative-position bias, ids the regions a cyclic shift glues together."""

    @staticmethod
    def forward(ctx, q, k, v, bias, mask, ids, scale):
        from . import attention as _attn

        add = _attn.Additive(q.shape[1], k.shape[1], bias, mask, ids)
        o, lse = _attn.fwd(q, k, v, False, scale, additive=add)
        ctx.scale, ctx.add = scale, add
        ctx.bias_dtype = bias.dtype if bias is not None else None
        ctx.save_for_backward(q, k, v, o, lse)
        return o

    @staticmethod
    def backward(ctx, do):
        from . import attention as _attn

        q, k, v, o, lse = ctx.saved_tensors
        add = ctx.add
        want_dbias = add.bias is not None and ctx.needs_input_grad[3]
        dbias = torch.zeros(add.bias.shape, dtype=torch.float32, device=q.device) if want_dbias else None
        dq, dk, dv = _attn.bwd(do, q, k, v, o, lse, False, ctx.scale, additive=add, dbias=dbias)
        if want_dbias:
            dbias = dbias[:, :, :add.sk].to(ctx.bias_dtype)
        return dq, dk, dv, dbias, None, None, None


def biased_attention(q, k, v, bias=None, mask=None, ids=None, scale: float | None = None):
    """Attention with additive bias / additive mask / group ids: the kernels for bf16 CUDA operands, PyTorch expressions
    otherwise."""
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    if bias is None and mask is None and ids is None:
        return attention(q, k, v, causal=False, scale=scale)[0]
    if Fn.biased_attention_native(q, k, v):
        return BiasedAttentionFn.apply(q, k, v, bias, mask, ids, scale)
    return Fn.biased_attention_reference(q, k, v, scale, bias, mask, ids)


class RopeFn(torch.autograd.Function):
    """Out-of-place rotary embedding on [tokens, heads, dh] (used by the Ulysses / ring paths)."""

    @staticmethod
    def forward(ctx, x, inv_freq, pos_div, pos_mod, pos_offset, positions):
        y = x.contiguous().clone()
        Fn.rope_(y, inv_freq, pos_div, pos_mod, pos_offset, positions, False)
        ctx.args = (pos_div, pos_mod, pos_offset)
        ctx.save_for_backward(inv_freq, positions)
        return y

    @staticmethod
    def backward(ctx, dy):
        inv_freq, positions = ctx.saved_tensors
        dx = dy.contiguous().clone()
        Fn.rope_(dx, inv_freq, *ctx.args, positions, True)
        return dx, None, None, None, None, None


def rope(x, inv_freq, pos_div=1, pos_mod=0, pos_offset=0, positions=None):
    return RopeFn.apply(x, inv_freq, pos_div, pos_mod, pos_offset, positions)


# --------------------------------------------------------------------------- embedding
class EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table, pos_ids, pos_table, vocab_start, group):
        out = Fn.embedding_fwd(ids, table, vocab_start, pos_ids if pos_table is not None else None, pos_table)
        if C.group_size(group) > 1:
            if pos_table is not None:
                raise ValueError("learned positions are added after the vocab-parallel reduction")
            C.all_reduce_(out, group)
        ctx.vocab_start = vocab_start
        ctx.save_for_backward(ids, table, pos_ids, pos_table)
        return out

    @staticmethod
    def backward(ctx, dout):
        ids, table, pos_ids, pos_table = ctx.saved_tensors
        dout = dout.contiguous()

        def table_grad(tbl, idx, start):
            def into(mg):
                if mg.dtype == torch.float32:
                    Fn.embedding_bwd(idx, dout, mg.view(tbl.shape), start)
                else:
                    tmp = torch.zeros(tbl.shape, dtype=torch.float32, device=tbl.device)
                    Fn.embedding_bwd(idx, dout, tmp, start)
                    mg.view(tbl.shape).add_(tmp.to(mg.dtype))

            def fresh():
                tmp = torch.zeros(tbl.shape, dtype=torch.float32, device=tbl.device)
                Fn.embedding_bwd(idx, dout, tmp, start)
                return tmp.to(tbl.dtype)

            return _accum_param_grad(tbl, into, fresh)

        dtable = table_grad(table, ids, ctx.vocab_start)
        dpos = table_grad(pos_table, pos_ids, 0) if pos_table is not None else None
        return None, dtable, None, dpos, None, None


def embedding(ids, table, pos_ids=None, pos_table=None, vocab_start: int = 0, group=None):
    return EmbeddingFn.apply(ids, table, pos_ids, pos_table, vocab_start, group)


# --------------------------------------------------------------------------- LM head + cross entropy
@dataclass(frozen=True)
class LossCfg:
    vocab_start: int = 0
    group: Any = None             # vocab-parallel group
    ignore_index: int = -100
    mode: str = "col"             # col (x replicated) | col_sp (x sequence-sharded over `group`)
    fp32_logits: bool = False     # keep the logits in fp32 (reference: --entropy_in_fp32)


class LMHeadLossFn(torch.autograd.Function):
    """Per-token cross entropy of ``x W^T`` against labels, vocab-parallel over ``cfg.group``.

    On bf16 CUDA tensors the head GEMM's epilogue computes the statistics from its fp32 accumulators and stores no
    logits at all; backward runs the GEMM once more with an epilogue that writes (softmax - onehot) * dloss. Otherwise
    forward keeps the logits and three fp32 statistics per row. Either way the cross-rank step is ONE
    all-gather of the packed (max, sum-exp, target-logit) triples instead of the reference's three
    all-reduces (megatron/core/tensor_parallel/cross_entropy.py:21-29,61-72,78-89). Backward turns the
    logits into (softmax - onehot) * dloss in place and feeds the two gradient GEMMs."""

    @staticmethod
    def forward(ctx, x, W, labels, cfg: LossCfg):
        n = C.group_size(cfg.group)
        x2 = x.reshape(-1, x.shape[-1])
        xg = C.all_gather_first_dim(x2, cfg.group) if (cfg.mode == "col_sp" and n > 1) else x2
        labels = labels.reshape(-1)
        fused = (not cfg.fp32_logits) and head_xent_supported(xg, W)
        if fused:
            # statistics straight from the GEMM's fp32 accumulators; no [tokens, vocab] tensor is ever written
            logits = None
            mx, se, tg = head_xent_stats(xg, W, labels, cfg.vocab_start, cfg.ignore_index)
        else:
            logits = gemm(xg, W, out_dtype=torch.float32 if (cfg.fp32_logits or not x.is_cuda) else None)
            mx, se, tg = Fn.xent_stats(logits, labels, cfg.vocab_start)
        if n > 1:
            packed = torch.stack([mx, se, tg], dim=0)
            allp = C.all_gather_first_dim(packed.unsqueeze(0), cfg.group)  # [n, 3, rows]
            gmx = allp[:, 0].max(dim=0).values
            se = (allp[:, 1] * torch.exp(allp[:, 0] - gmx.unsqueeze(0))).sum(0)
            tg = allp[:, 2].sum(0)
            mx = gmx
        keep = (labels != cfg.ignore_index)
        loss = (torch.log(se) + mx - tg) * keep.to(torch.float32)
        ctx.cfg, ctx.n, ctx.fused = cfg, n, fused
        ctx.x_shape = x.shape
        if fused:
            ctx.save_for_backward(x2, W, labels, mx, se)
        else:
            ctx.save_for_backward(x2, W, labels, logits, mx, se, tg)
        return loss

    @staticmethod
    def backward(ctx, dloss):
        cfg, n = ctx.cfg, ctx.n
        if ctx.fused:
            x2, W, labels, mx, se = ctx.saved_tensors
            xg = C.all_gather_first_dim(x2, cfg.group) if (cfg.mode == "col_sp" and n > 1) else x2
            keep = (labels != cfg.ignore_index).to(torch.float32)
            # the head GEMM runs once more; its epilogue turns each fp32 logit into its gradient
            dlog = head_xent_grad(xg, W, labels, torch.log(se) + mx, dloss.reshape(-1).float() * keep, cfg.vocab_start,
                                  cfg.ignore_index)
        else:
            x2, W, labels, logits, mx, se, tg = ctx.saved_tensors
            Fn.xent_loss_grad_(logits, labels, mx, se, tg, 1.0, cfg.vocab_start, cfg.ignore_index,
                               scale_tensor=dloss.contiguous().float())
            dlog = logits if logits.dtype == x2.dtype else logits.to(x2.dtype)
            xg = C.all_gather_first_dim(x2, cfg.group) if (cfg.mode == "col_sp" and n > 1) else x2
        dx = gemm(dlog, W, b_mn=True)
        if n > 1:
            dx = C.reduce_scatter_first_dim(dx, cfg.group) if cfg.mode == "col_sp" else C.all_reduce_(dx, cfg.group)
        dW = _wgrad(W, dlog, xg)
        return dx.view(ctx.x_shape), dW, None, None


def lm_head_loss(x, W, labels, cfg: LossCfg = LossCfg()):
    return LMHeadLossFn.apply(x, W, labels, cfg)
