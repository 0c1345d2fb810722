"""Context parallelism with the zigzag sequence split (rank c of cp owns chunks c and 2cp-1-c of 2cp).

Reference: zigzag ring FlashAttention, galvatron/core/runtime/tensor_parallel/transformer.py:2252-2680, which
circulates K/V blocks with batched isend/irecv and merges partial outputs by log-sum-exp. The ``nccl``
implementation here gathers the K/V shards of the cp group once, reorders them to global order and runs the
attention kernel once per local query chunk: query chunk g (global index) attends causally to the first g+1
key chunks (the kernel aligns the last query with the last key). The exchanged volume equals the ring's; dK/dV
return with one reduce-scatter. The result is identical to attention over the full sequence.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import autograd as A
from . import collectives as C


class _GatherKV(torch.autograd.Function):
    """[s_loc, b, c] -> [s, b, c] in global sequence order over the zigzag cp group; backward reduce-scatters."""

    @staticmethod
    def forward(ctx, x, cp, group, impl="nccl"):
        if impl == "fused" and x.is_cuda and x.dtype == torch.bfloat16 and x.numel() % 8 == 0:
            # every rank pulls the other ranks' KV rows straight from their (peer-mapped) memory
            from . import fused
            parts = fused.allgather_pull(x.contiguous(), fused.comm_group(group), "cp_kv").view(cp, *x.shape)
        else:
            parts = C.all_gather_first_dim(x.contiguous().unsqueeze(0), group)  # [cp, s_loc, b, c]
        s_loc = x.shape[0]
        half = s_loc // 2
        early = parts[:, :half]                                                    # chunk r
        late = parts[:, half:].flip(0)                                             # chunk 2cp-1-r, r descending
        ctx.cp, ctx.group, ctx.half = cp, group, half
        return torch.cat([early.reshape(cp * half, *x.shape[1:]), late.reshape(cp * half, *x.shape[1:])], 0)

    @staticmethod
    def backward(ctx, dy):
        cp, half = ctx.cp, ctx.half
        early = dy[: cp * half].reshape(cp, half, *dy.shape[1:])
        late = dy[cp * half:].reshape(cp, half, *dy.shape[1:]).flip(0)
        parts = torch.cat([early, late], dim=1).contiguous()                      # [cp, s_loc, b, c]
        out = torch.empty(parts.shape[1:], dtype=dy.dtype, device=dy.device)
        dist.reduce_scatter_tensor(out, parts.view(-1, *parts.shape[2:]), group=ctx.group)
        return out, None, None, None


def ring_attention_packed(qkv: torch.Tensor, attn_module, ctx, causal: bool, rope: bool) -> torch.Tensor:
    st, cfg = attn_module.st, attn_module.cfg
    cp, r = st.cp, st.cp_rank
    group = st.cp_group.group
    hq, hk, dh = attn_module.hq_w, attn_module.hk_w, cfg.head_dim
    b = ctx.batch
    s_loc = qkv.shape[0] // b
    half = s_loc // 2
    chunk = half
    x = qkv.view(s_loc, b, (hq + 2 * hk) * dh)
    q = x[..., : hq * dh].reshape(s_loc, b, hq, dh)
    k = x[..., hq * dh:(hq + hk) * dh].reshape(s_loc, b, hk, dh)
    v = x[..., (hq + hk) * dh:].reshape(s_loc, b, hk, dh)
    if rope:
        pos_s = torch.cat([torch.arange(r * chunk, (r + 1) * chunk, device=qkv.device),
                           torch.arange((2 * cp - 1 - r) * chunk, (2 * cp - r) * chunk, device=qkv.device)])
        positions = pos_s.view(s_loc, 1).expand(s_loc, b).reshape(-1)
        q = A.rope(q.reshape(s_loc * b, hq, dh), attn_module.inv_freq, 1, 0, 0, positions).view(s_loc, b, hq, dh)
        k = A.rope(k.reshape(s_loc * b, hk, dh), attn_module.inv_freq, 1, 0, 0, positions).view(s_loc, b, hk, dh)
    kv = torch.cat([k.reshape(s_loc, b, hk * dh), v.reshape(s_loc, b, hk * dh)], dim=-1)
    kv_all = _GatherKV.apply(kv, cp, group, st.impl)                                        # [s, b, 2 hk dh], global order
    k_all = kv_all[..., : hk * dh].reshape(-1, b, hk, dh).transpose(0, 1)
    v_all = kv_all[..., hk * dh:].reshape(-1, b, hk, dh).transpose(0, 1)
    outs = []
    for qi, g in ((0, r), (1, 2 * cp - 1 - r)):
        qc = q[qi * half:(qi + 1) * half].transpose(0, 1)                          # [b, chunk, hq, dh]
        if causal:
            kend = (g + 1) * chunk
            o, _ = A.attention(qc, k_all[:, :kend], v_all[:, :kend], True, None)
        else:
            o, _ = A.attention(qc, k_all, v_all, False, None)
        outs.append(o.transpose(0, 1))                                             # [chunk, b, hq, dh]
    return torch.cat(outs, 0).reshape(s_loc * b, hq * dh)
