"""Seeding, a distributed dataloader helper and loss printing (reference: galvatron/utils/training_utils.py:7-40)."""
from __future__ import annotations

import random

import numpy as np
import torch


def set_seed(seed: int = 1234) -> None:
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def distributed_dataloader(dataset, global_bsz: int, shuffle: bool = True, args=None, group=None, collate_fn=None, model=None):
    """A DataLoader whose sampler splits the dataset over the data-parallel ``group``; every rank of the
    group draws ``global_bsz / group_size`` samples per step. With ``model`` (a ``GalvatronModel``) the split follows the
    model's data layout instead: ranks that share a tensor-, sequence- or context-parallel group draw the same samples."""
    import torch.distributed as dist
    from torch.utils.data import DataLoader
    from torch.utils.data.distributed import DistributedSampler

    if group is not None and hasattr(group, "num_replicas"):        # model.dp_groups_whole[i].group
        sampler = DistributedSampler(dataset, shuffle=shuffle, num_replicas=group.num_replicas, rank=group.rank)
        return DataLoader(dataset, batch_size=global_bsz // group.num_replicas, sampler=sampler, collate_fn=collate_fn)
    if model is not None:
        per = model.local_batch_size()
        sampler = DistributedSampler(dataset, shuffle=shuffle, num_replicas=global_bsz // per, rank=model.batch_slice()[0] // per)
        return DataLoader(dataset, batch_size=per, sampler=sampler, collate_fn=collate_fn)
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    pp_deg = getattr(args, "pp_deg", 1) if args is not None else 1
    dp_world = max(world // pp_deg, 1) if group is None else world
    dp_rank = rank % dp_world
    sampler = DistributedSampler(dataset, shuffle=shuffle, num_replicas=dp_world, rank=dp_rank)
    return DataLoader(dataset, batch_size=global_bsz // dp_world, sampler=sampler, collate_fn=collate_fn)


def print_loss(args, loss, ep: int, it: int) -> None:
    """Print the loss from the rank(s) that own it: rank 0 without pipeline, the last stage otherwise."""
    import torch.distributed as dist

    if loss is None:
        return
    rank = dist.get_rank() if dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_initialized() else 1
    pp_deg = getattr(args, "pp_deg", 1)
    owner = 0 if pp_deg <= 1 else world - 1
    if rank == owner:
        if isinstance(loss, (list, tuple)):
            loss = sum(float(x) for x in loss) / max(len(loss), 1)
        print("[Epoch %d] (Iteration %d): Loss = %.6f" % (ep, it, float(loss)), flush=True)
