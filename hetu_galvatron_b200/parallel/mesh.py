"""Rank layout and process-group factory.

Layout (same as the reference's comm-group factory, galvatron/core/runtime/comm_groups.py:71-236):
pipeline stages are contiguous blocks of ``world / pp`` ranks; inside a stage the tensor- (or Ulysses
sequence-) parallel ranks are consecutive, context-parallel ranks are strided by ``tp``, data-parallel ranks
are strided by ``tp * cp``. On one NVSwitch box every peer is equally near, so the reference's
"strided TP" variant (tp_consecutive_flag = 0) is accepted in plans but laid out consecutively.

``new_group`` is a collective over the whole world, so groups are created per *signature* (kind, tp, cp):
the first request for a signature creates every group of that signature on every rank, in a fixed order.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch.distributed as dist


@dataclass
class CommGroup:
    ranks: List[int]
    group: object = None  # torch ProcessGroup (None for single-rank groups or single-process runs)

    @property
    def size(self) -> int:
        return len(self.ranks)

    def has_rank(self, rank: int) -> bool:
        return rank in self.ranks

    def rank_in_group(self, rank: int) -> int:
        return self.ranks.index(rank)

    def print(self) -> None:
        print(self.ranks, end=" ")


class Mesh:
    def __init__(self, world_size: Optional[int] = None, rank: Optional[int] = None, pp_deg: int = 1):
        if world_size is None:
            world_size = dist.get_world_size() if dist.is_initialized() else 1
        if rank is None:
            rank = dist.get_rank() if dist.is_initialized() else 0
        assert world_size % pp_deg == 0, "world size must be divisible by pp_deg"
        self.world_size, self.rank, self.pp_deg = world_size, rank, pp_deg
        self.stage_size = world_size // pp_deg
        self.stage = rank // self.stage_size
        self.local = rank % self.stage_size
        self._cache: Dict[Tuple, CommGroup] = {}

    # ------------------------------------------------------------------ rank lists
    def _stage_base(self, stage: int) -> int:
        return stage * self.stage_size

    def tp_ranks(self, tp: int, stage: int, block: int) -> List[int]:
        base = self._stage_base(stage) + block * tp
        return list(range(base, base + tp))

    def enumerate_groups(self, kind: str, tp: int = 1, cp: int = 1) -> List[List[int]]:
        """Every group of a signature, over all stages, in creation order."""
        S, out = self.stage_size, []
        if kind == "pp":
            return [[s * S + i for s in range(self.pp_deg)] for i in range(S)]
        if kind == "embed":
            if self.pp_deg == 1:
                return [[i] for i in range(S)]
            return [[i, (self.pp_deg - 1) * S + i] for i in range(S)]
        if kind == "world":
            return [list(range(self.world_size))]
        for s in range(self.pp_deg):
            base = self._stage_base(s)
            if kind == "stage":
                out.append(list(range(base, base + S)))
            elif kind == "tp":
                assert S % tp == 0
                out += [list(range(base + b * tp, base + (b + 1) * tp)) for b in range(S // tp)]
            elif kind == "cp":
                blk = tp * cp
                assert S % blk == 0
                for b in range(S // blk):
                    for t in range(tp):
                        out.append([base + b * blk + c * tp + t for c in range(cp)])
            elif kind == "tpcp":  # the tp x cp block (sequence is split over all of it)
                blk = tp * cp
                out += [list(range(base + b * blk, base + (b + 1) * blk)) for b in range(S // blk)]
            elif kind == "dp":
                blk = tp * cp
                assert S % blk == 0
                for i in range(blk):
                    out.append([base + i + d * blk for d in range(S // blk)])
            elif kind == "wdp":
                # Weight-replica group = the ranks that hold the same weight shard: gradients are reduced and
                # ZeRO shards are spread over it. `tp` here is the WEIGHT sharding degree: the Megatron-TP
                # degree, or 1 for Ulysses layers (full weights on every rank of the sp group). Context-parallel
                # ranks replicate weights too, so they are part of it.
                out += [[base + t + j * tp for j in range(S // tp)] for t in range(tp)]
            else:
                raise ValueError(kind)
        return out

    # ------------------------------------------------------------------ groups
    def group(self, kind: str, tp: int = 1, cp: int = 1) -> CommGroup:
        key = (kind, tp if kind not in ("pp", "embed", "world", "stage") else 0,
               cp if kind in ("cp", "dp", "tpcp") else 0)
        if key in self._cache:
            return self._cache[key]
        mine = None
        for ranks in self.enumerate_groups(kind, tp, cp):
            pg = None
            if dist.is_initialized() and len(ranks) > 1 and self.world_size > 1:
                pg = dist.new_group(ranks)
            if self.rank in ranks:
                mine = CommGroup(ranks, pg)
        assert mine is not None
        self._cache[key] = mine
        if mine.group is not None:
            from . import fused
            fused.register_group(mine)      # the fused kernels need the rank list behind a ProcessGroup
        return mine

    def pp_prev_next(self) -> Tuple[Optional[int], Optional[int]]:
        prev = self.rank - self.stage_size if self.stage > 0 else None
        nxt = self.rank + self.stage_size if self.stage < self.pp_deg - 1 else None
        return prev, nxt

    # coordinates of this rank inside a (tp, cp) layer layout
    def coords(self, tp: int, cp: int = 1) -> Dict[str, int]:
        blk = tp * cp
        return {"tp": self.local % tp, "cp": (self.local % blk) // tp, "dp": self.local // blk,
                "dp_size": self.stage_size // blk}


def gen_comm_groups(all_tp_sizes, all_sp_sizes, all_cp_sizes, pp_size, tp_consecutive_flags=None, show_rank=-1,
                    mesh: Optional[Mesh] = None):
    """Per-layer group lists in the shape the reference returns them (comm_groups.py:416-569):
    (pp_group, tp_groups, sp_groups, cp_groups, dp_groups, seq_data_groups, embedding_group, ...).
    ``all_tp_sizes[i]`` / ``all_sp_sizes[i]`` are the Megatron-TP and Ulysses-SP degrees of layer i (at most one
    of them is > 1)."""
    mesh = mesh or Mesh(pp_deg=pp_size)
    tp_groups, sp_groups, cp_groups, dp_groups, sdp_groups = [], [], [], [], []
    for tp, sp, cp in zip(all_tp_sizes, all_sp_sizes, all_cp_sizes):
        assert tp == 1 or sp == 1, "a layer uses Megatron-TP or Ulysses-SP, not both"
        width = max(tp, sp)
        tp_groups.append(mesh.group("tp", tp))
        sp_groups.append(mesh.group("tp", sp))
        cp_groups.append(mesh.group("cp", width, cp))
        dp_groups.append(mesh.group("dp", width, cp))
        sdp_groups.append(mesh.group("wdp", tp))
    pp_group = mesh.group("pp")
    embedding_group = mesh.group("embed")
    if show_rank in (mesh.rank, 0) and show_rank >= 0 and mesh.rank == show_rank:
        print("pp group:", pp_group.ranks)
        for i, (t, s, c, d) in enumerate(zip(tp_groups, sp_groups, cp_groups, dp_groups)):
            print("layer %d: tp %s sp %s cp %s dp %s" % (i, t.ranks, s.ranks, c.ranks, d.ranks))
    return pp_group, tp_groups, sp_groups, cp_groups, dp_groups, sdp_groups, embedding_group, mesh
