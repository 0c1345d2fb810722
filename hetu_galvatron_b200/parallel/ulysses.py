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
from . import collectives as C


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


def ulysses_attention(qkv: torch.Tensor, attn_module, ctx, causal: bool, rope: bool) -> torch.Tensor:
    st, cfg = attn_module.st, attn_module.cfg
    p, group = st.tp, st.pg()
    hq, hk, dh = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    idx = getattr(attn_module, "_ulysses_idx", None)
    if idx is None or idx.device != qkv.device:
        idx = _send_columns(hq, hk, dh, p, qkv.device)
        attn_module._ulysses_idx = idx
    if st.impl == "fused" and qkv.is_cuda:
        from . import fused
        full = fused.seq_to_heads(qkv, idx, st.tp_group)
    else:
        full = _ColsToRanks.apply(qkv, idx, group)              # [s * b, (hq/p + 2 hk_loc) * dh]
    acfg = A.AttnCfg(batch=ctx.batch, hq=hq // p, hk=max(hk // p, 1), dh=dh, causal=causal, rope=rope)
    o = A.packed_attention(full, acfg, attn_module.inv_freq, None)   # [s * b, hq/p * dh]
    if st.impl == "fused" and qkv.is_cuda:
        from . import fused
        return fused.heads_to_seq(o, p, st.tp_group)
    return _RowsToRanks.apply(o, p, group)                       # [s_loc * b, hq * dh]
