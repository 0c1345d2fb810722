"""Group-explicit collectives over ``torch.distributed`` (NCCL on GPUs, gloo on CPU ranks).

These are the plain-library implementations of every communication step of the runtime (the
reference's only implementation: megatron/core/tensor_parallel/mappings_group.py:11-250). The fused
peer-memory kernels in ``parallel/fused.py`` replace them on the hot paths and are validated
against them.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def group_size(group) -> int:
    if group is None or not dist.is_initialized():
        return 1
    return dist.get_world_size(group)


def group_rank(group) -> int:
    if group is None or not dist.is_initialized():
        return 0
    return dist.get_rank(group)


def all_gather_first_dim(x: torch.Tensor, group) -> torch.Tensor:
    n = group_size(group)
    if n == 1:
        return x
    x = x.contiguous()
    out = torch.empty((n * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x, group=group)
    return out


def reduce_scatter_first_dim(x: torch.Tensor, group) -> torch.Tensor:
    n = group_size(group)
    if n == 1:
        return x
    x = x.contiguous()
    out = torch.empty((x.shape[0] // n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.reduce_scatter_tensor(out, x, group=group)
    return out


def all_reduce_(x: torch.Tensor, group, op=None) -> torch.Tensor:
    if group_size(group) > 1:
        dist.all_reduce(x, op=op or dist.ReduceOp.SUM, group=group)
    return x


def all_gather_last_dim(x: torch.Tensor, group) -> torch.Tensor:
    n = group_size(group)
    if n == 1:
        return x
    parts = [torch.empty_like(x) for _ in range(n)]
    dist.all_gather(parts, x.contiguous(), group=group)
    return torch.cat(parts, dim=-1)


def all_to_all_single(out: torch.Tensor, inp: torch.Tensor, group) -> torch.Tensor:
    dist.all_to_all_single(out, inp.contiguous(), group=group)
    return out


def broadcast_(x: torch.Tensor, src_global_rank: int, group) -> torch.Tensor:
    if group_size(group) > 1:
        dist.broadcast(x, src=src_global_rank, group=group)
    return x
