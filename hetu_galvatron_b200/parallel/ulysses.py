"""Ulysses sequence parallelism: sequence-sharded activations, head-sharded attention.

Reference: galvatron/core/runtime/tensor_parallel/transformer.py:1904-2177 (``single_all_to_all``,
``_SeqAllToAll``, ``DistributedAttention``): q, k and v each take one all-to-all, the attention output a
fourth. Here the packed QKV projection output takes ONE all-to-all (q, k and v columns of the destination's
head group are packed together), and thanks to the sequence-major token order the received blocks are already
the full sequence in order, so no permute/copy is needed on the receive side. RoPE is applied after the
exchange, on full-sequence positions. GQA with fewer KV heads than ranks replicates KV heads on the send
side (their gradients are summed on the way back).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import autograd as A


class _ColsToRanks(torch.autograd.Function):
    """[rows_local, cols] -> [p * rows_local, c]: rank j receives columns ``idx[j]`` of every rank's rows."""

    @staticmethod
    def forward(ctx, x, idx, group):
        p, c = idx.shape
        rows = x.shape[0]
        send = x.index_select(1, idx.reshape(-1)).view(rows, p, c).permute(1, 0, 2).contiguous()
        out = torch.empty(p * rows, c, dtype=x.dtype, device=x.device)
        dist.all_to_all_single(out, send.view(p * rows, c), group=group)
        ctx.group, ctx.cols = group, x.shape[1]
        ctx.save_for_backward(idx)
        return out

    @staticmethod
    def backward(ctx, dy):
        (idx,) = ctx.saved_tensors
        p, c = idx.shape
        rows = dy.shape[0] // p
        send = dy.contiguous().view(p, rows, c)
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=ctx.group)
        g = recv.permute(1, 0, 2).reshape(rows, p * c)
        dx = torch.zeros(rows, ctx.cols, dtype=dy.dtype, device=dy.device)
        dx.index_add_(1, idx.reshape(-1), g)
        return dx, None, None


class _RowsToRanks(torch.autograd.Function):
    """[p * rows_local, c] -> [rows_local, p * c]: rank i receives row block i of every rank, side by side."""

    @staticmethod
    def forward(ctx, x, p, group):
        rows, c = x.shape[0] // p, x.shape[1]
        send = x.contiguous().view(p, rows, c)
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=group)
        ctx.group, ctx.p = group, p
        return recv.permute(1, 0, 2).reshape(rows, p * c)

    @staticmethod
    def backward(ctx, dy):
        p = ctx.p
        rows, pc = dy.shape
        c = pc // p
        send = dy.view(rows, p, c).permute(1, 0, 2).contiguous()
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=ctx.group)
        return recv.view(p * rows, c), None, None


def _exchange_blocks(send: torch.Tensor, cg, tag: str) -> torch.Tensor:
    """All-to-all of equal blocks ([p, ...]: block j goes to rank j) for the backward halves of the fused Ulysses
    paths: this package's pull kernel over peer memory (``gv_alltoall_pull``) instead of ``all_to_all_single``."""
    from . import fused

    if send.is_cuda and send.dtype == torch.bfloat16 and (send.numel() // cg.size * 2) % 16 == 0:
        return fused.alltoall_pull(send.contiguous(), cg, tag)
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send.contiguous(), group=cg.group)
    return recv


def _send_columns(hq: int, hk: int, dh: int, p: int, device) -> torch.Tensor:
    """Column indices of the packed [q | k | v] projection that go to each rank: [p, (hq/p + 2*hk_loc) * dh]."""
    hq_loc = hq // p
    hk_loc = max(hk // p, 1)
    cols = []
    for j in range(p):
        q_heads = list(range(j * hq_loc, (j + 1) * hq_loc))
        if hk >= p:
            kv_heads = list(range(j * hk_loc, (j + 1) * hk_loc))
        else:
            kv_heads = [j * hk // p]     # KV head shared by this rank's query heads
        c = []
        for h in q_heads:
            c += range(h * dh, (h + 1) * dh)
        for h in kv_heads:
            c += range((hq + h) * dh, (hq + h + 1) * dh)
        for h in kv_heads:
            c += range((hq + hk + h) * dh, (hq + hk + h + 1) * dh)
        cols.append(c)
    return torch.tensor(cols, dtype=torch.int64, device=device)


class UlyssesQKVFn(torch.autograd.Function):
    """Fused path: QKV projection + sequence -> head exchange in one GEMM (epilogue stores to the owning ranks)."""

    @staticmethod
    def forward(ctx, x, W, bias, idx, cg):
        from . import fused
        x2 = x.reshape(-1, x.shape[-1])
        full = fused.qkv_to_heads(x2, W, bias, idx, cg)
        ctx.cg = cg
        ctx.save_for_backward(x2, W, bias, idx)
        return full

    @staticmethod
    def backward(ctx, dfull):
        from ..ops.autograd import _vec_grad, _wgrad
        from ..ops import functional as Fn
        from ..ops.gemm import gemm
        x2, W, bias, idx = ctx.saved_tensors
        p, c = idx.shape
        rows = dfull.shape[0] // p
        recv = _exchange_blocks(dfull.contiguous().view(p, rows, c), ctx.cg, "u1b")
        g = recv.permute(1, 0, 2).reshape(rows, p * c)
        dqkv = torch.zeros(rows, W.shape[0], dtype=dfull.dtype, device=dfull.device)
        dqkv.index_add_(1, idx.reshape(-1), g)
        dx = gemm(dqkv, W, b_mn=True)
        dW = _wgrad(W, dqkv, x2)
        db = _vec_grad(bias, lambda buf: Fn.colsum_accum(dqkv, buf)) if bias is not None else None
        return dx, dW, db, None, None


class UlyssesOutFn(torch.autograd.Function):
    """Fused path: head -> sequence exchange + output projection in one GEMM (A K-slices read from their owners)."""

    @staticmethod
    def forward(ctx, o, W, bias, residual, cg):
        from . import fused
        y = fused.heads_to_out(o, W, bias, residual, cg)
        ctx.cg, ctx.has_res = cg, residual is not None
        ctx.save_for_backward(o, W, bias)
        return y

    @staticmethod
    def backward(ctx, dy):
        from ..ops.autograd import _vec_grad, _wgrad
        from ..ops import functional as Fn
        from ..ops.gemm import gemm
        o, W, bias = ctx.saved_tensors
        p = ctx.cg.size
        dy2 = dy.reshape(-1, W.shape[0]).contiguous()
        rows_loc, c_o = o.shape[0] // p, o.shape[1]
        # this rank's rows of every rank's heads, side by side: [rows_loc, hq * dh]
        a_full = _exchange_blocks(o.contiguous().view(p, rows_loc, c_o), ctx.cg, "u2b_o").permute(1, 0, 2).reshape(rows_loc, p * c_o)
        da = gemm(dy2, W, b_mn=True)
        dW = _wgrad(W, dy2, a_full)
        rows, pc = da.shape
        c = pc // p
        recv = _exchange_blocks(da.view(rows, p, c).permute(1, 0, 2).contiguous(), ctx.cg, "u2b_da")
        db = _vec_grad(bias, lambda buf: Fn.colsum_accum(dy2, buf)) if bias is not None else None
        return recv.view(p * rows, c), dW, db, (dy if ctx.has_res else None), None


def _dropout(attn_module, ctx, heads_local: int):
    """Attention-probability dropout of this rank's head group (global head indices keep the mask layout-independent)."""
    from ..models.transformer import attention_dropout_spec

    return attention_dropout_spec(attn_module.cfg, ctx, attn_module.layer_idx, attn_module.st.tp_rank * heads_local)


def ulysses_block_fused(x, residual, attn_module, ctx, causal: bool, rope: bool) -> torch.Tensor:
    """norm output -> [fused QKV + exchange] -> attention on full sequence / local heads -> [fused exchange + out-proj]."""
    st, cfg = attn_module.st, attn_module.cfg
    p = st.tp
    hq, hk, dh = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    idx = getattr(attn_module, "_ulysses_idx", None)
    if idx is None or idx.device != x.device:
        idx = _send_columns(hq, hk, dh, p, x.device)
        attn_module._ulysses_idx = idx
    full = UlyssesQKVFn.apply(x, attn_module.wqkv, attn_module.bqkv, idx, st.tp_group)
    acfg = A.AttnCfg(batch=ctx.batch, hq=hq // p, hk=max(hk // p, 1), dh=dh, causal=causal, rope=rope,
                     dropout=_dropout(attn_module, ctx, hq // p))
    o = A.packed_attention(full, acfg, attn_module.inv_freq, None)
    return UlyssesOutFn.apply(o, attn_module.wo, attn_module.bo, residual, st.tp_group)


def ulysses_attention(qkv: torch.Tensor, attn_module, ctx, causal: bool, rope: bool) -> torch.Tensor:
    st, cfg = attn_module.st, attn_module.cfg
    p, group = st.tp, st.pg()
    hq, hk, dh = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    idx = getattr(attn_module, "_ulysses_idx", None)
    if idx is None or idx.device != qkv.device:
        idx = _send_columns(hq, hk, dh, p, qkv.device)
        attn_module._ulysses_idx = idx
    full = _ColsToRanks.apply(qkv, idx, group)                  # [s * b, (hq/p + 2 hk_loc) * dh]
    acfg = A.AttnCfg(batch=ctx.batch, hq=hq // p, hk=max(hk // p, 1), dh=dh, causal=causal, rope=rope,
                     dropout=_dropout(attn_module, ctx, hq // p))
    o = A.packed_attention(full, acfg, attn_module.inv_freq, None)   # [s * b, hq/p * dh]
    return _RowsToRanks.apply(o, p, group)                       # [s_loc * b, hq * dh]
