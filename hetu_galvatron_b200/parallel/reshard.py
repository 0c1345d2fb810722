"""Activation redistribution between adjacent modules that use different parallel layouts.

A layout says how a stage's micro-batch ``[seq, B, hidden]`` is spread over the stage's ranks: the batch is split
over ``dp = stage_size / (tp * cp)`` groups, the sequence over ``cp`` ranks (zigzag: rank c owns chunks c and
2cp-1-c of 2cp, reference galvatron/core/runtime/redistribute.py:8-44) and, when the layer is sequence parallel,
further over the ``tp`` ranks; otherwise the tp ranks hold replicas.

Two implementations sit behind ``redistribute``:
* ``nccl``: all-gather of every rank's piece over the stage group, then a local gather of the rows the new
  layout needs (the reference's algorithm family: redistribute.py:269-350 all-gathers over the old group and
  slices);
* ``fused``: one kernel in which the destination rank reads exactly the rows it needs from its peers' buffers
  (``parallel/fused.py``), no intermediate full tensor.
Integer tensors (labels, masks) take the same path; their backward is None.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

import torch

from .collectives import all_gather_first_dim
from .mesh import Mesh


@dataclass(frozen=True)
class Layout:
    tp: int = 1
    cp: int = 1
    seq_sharded: bool = False   # sequence split over the tp ranks (Megatron-SP or Ulysses)

    def block(self) -> int:
        return self.tp * self.cp

    def dp(self, stage_size: int) -> int:
        return stage_size // self.block()

    def seq_parts(self) -> int:
        return self.cp * (self.tp if self.seq_sharded else 1)


def seq_positions(layout: Layout, local_rank: int, seq: int) -> torch.Tensor:
    """Global sequence positions held by ``local_rank`` (index inside its stage), in local order."""
    tp_idx = local_rank % layout.tp
    cp_idx = (local_rank % layout.block()) // layout.tp
    if layout.cp > 1:
        chunk = seq // (2 * layout.cp)
        a = torch.arange(cp_idx * chunk, (cp_idx + 1) * chunk)
        b = torch.arange((2 * layout.cp - 1 - cp_idx) * chunk, (2 * layout.cp - cp_idx) * chunk)
        pos = torch.cat([a, b])
    else:
        pos = torch.arange(seq)
    if layout.seq_sharded and layout.tp > 1:
        n = pos.numel() // layout.tp
        pos = pos[tp_idx * n:(tp_idx + 1) * n]
    return pos


def batch_range(layout: Layout, local_rank: int, stage_size: int, stage_batch: int) -> Tuple[int, int]:
    dp = layout.dp(stage_size)
    dp_idx = local_rank // layout.block()
    per = stage_batch // dp
    return dp_idx * per, (dp_idx + 1) * per


def source_map(old: Layout, new: Layout, local_rank: int, stage_size: int, stage_batch: int, seq: int):
    """For the destination ``local_rank`` under ``new``: for every (row of new local sequence, batch column) the
    owning source rank under ``old`` and the row/column inside that rank's piece. Returns int64 tensors
    (src_rank [s_new, b_new], src_row [s_new], src_col [b_new]) -- the row's owner does not depend on the column
    except through the dp index, so owner = row_owner_base[s] + col_owner[b] * old.block()."""
    pos_new = seq_positions(new, local_rank, seq)
    b_lo, b_hi = batch_range(new, local_rank, stage_size, stage_batch)
    # position -> (owner offset inside an old block, row inside the owner) for the old layout
    owner_in_block = torch.empty(seq, dtype=torch.int64)
    row_in_owner = torch.empty(seq, dtype=torch.int64)
    my_tp_old = local_rank % old.tp
    for r in range(old.block()):
        if not old.seq_sharded and (r % old.tp) != (my_tp_old % old.tp):
            continue  # replicas: read from the replica with my own tp index (any would do)
        p = seq_positions(old, r, seq)
        owner_in_block[p] = r
        row_in_owner[p] = torch.arange(p.numel())
    per_old = stage_batch // old.dp(stage_size)
    cols = torch.arange(b_lo, b_hi)
    col_owner_dp = cols // per_old
    col_in_owner = cols % per_old
    row_owner = owner_in_block[pos_new]
    src_rank = row_owner.view(-1, 1) + col_owner_dp.view(1, -1) * old.block()
    return src_rank, row_in_owner[pos_new], col_in_owner


def _redistribute_nccl(x3: torch.Tensor, old: Layout, new: Layout, mesh: Mesh, stage_batch: int, seq: int) -> torch.Tensor:
    """x3: [s_old_local, b_old_local, h] -> [s_new_local, b_new_local, h]."""
    S = mesh.stage_size
    if S == 1 or old == new:
        return x3
    grp = mesh.group("stage")
    parts = all_gather_first_dim(x3.contiguous().unsqueeze(0), grp.group)
    src_rank, src_row, src_col = source_map(old, new, mesh.local, S, stage_batch, seq)
    dev = x3.device
    src_rank, src_row, src_col = src_rank.to(dev), src_row.to(dev), src_col.to(dev)
    return parts[src_rank, src_row.view(-1, 1), src_col.view(1, -1)]


class _Redistribute(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2, b_old, old, new, mesh, stage_batch, seq, impl):
        ctx.args = (old, new, mesh, stage_batch, seq, impl)
        h = x2.shape[-1]
        s_old = x2.shape[0] // b_old
        x3 = x2.reshape(s_old, b_old, h)
        y3 = _dispatch(x3, old, new, mesh, stage_batch, seq, impl)
        ctx.b_new = y3.shape[1]
        return y3.reshape(-1, h)

    @staticmethod
    def backward(ctx, dy2):
        old, new, mesh, stage_batch, seq, impl = ctx.args
        h = dy2.shape[-1]
        dy3 = dy2.reshape(-1, ctx.b_new, h)
        dx3 = _dispatch(dy3, new, old, mesh, stage_batch, seq, impl)
        return dx3.reshape(-1, h), None, None, None, None, None, None, None


def _dispatch(x3, old, new, mesh, stage_batch, seq, impl):
    if impl == "fused" and x3.is_cuda and x3.dtype == torch.bfloat16 and 1 < mesh.stage_size <= 8 and x3.shape[-1] % 8 == 0:
        from . import fused
        return fused.reshard(x3, old, new, mesh, stage_batch, seq)
    return _redistribute_nccl(x3, old, new, mesh, stage_batch, seq)


def redistribute(x2: torch.Tensor, b_old: int, old: Layout, new: Layout, mesh: Mesh, stage_batch: int, seq: int,
                 impl: str = "nccl") -> Tuple[torch.Tensor, int]:
    """Relayout a sequence-major activation ``[s_old * b_old, h]``; returns (tensor, new local batch)."""
    b_new = stage_batch // new.dp(mesh.stage_size)
    if old == new or mesh.stage_size == 1:
        return x2, b_old
    if x2.is_floating_point() and x2.requires_grad:
        return _Redistribute.apply(x2, b_old, old, new, mesh, stage_batch, seq, impl), b_new
    h = x2.shape[-1]
    y3 = _dispatch(x2.reshape(-1, b_old, h), old, new, mesh, stage_batch, seq, "nccl" if not x2.is_floating_point() else impl)
    return y3.reshape(-1, h), b_new


def redistribute_batch_only(t: torch.Tensor, old: Layout, new: Layout, mesh: Mesh, stage_batch: int) -> torch.Tensor:
    """Labels / masks ``[b_old_local, ...]``: move along the batch dimension only (redistribute.py:231-267)."""
    S = mesh.stage_size
    if S == 1 or old.dp(S) == new.dp(S) and old.block() == new.block():
        return t
    grp = mesh.group("stage")
    parts = all_gather_first_dim(t.contiguous().unsqueeze(0), grp.group)
    per_old = stage_batch // old.dp(S)
    lo, hi = batch_range(new, mesh.local, S, stage_batch)
    cols = torch.arange(lo, hi, device=t.device)
    owner = (cols // per_old) * old.block()
    return parts[owner, cols % per_old]
