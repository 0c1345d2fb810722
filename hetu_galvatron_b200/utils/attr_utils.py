"""Dotted-path attribute access on nested objects (reference: galvatron/core/runtime/utils.py:22-45
``rgetattr / rsetattr / rhasattr``), plus the small helpers the reference keeps beside them."""
from __future__ import annotations

import functools

import torch


def rgetattr(obj, path: str, *default):
    """``rgetattr(m, "a.b.c")`` is ``m.a.b.c``; an empty path returns ``obj``; a default may be given like getattr."""
    if path == "":
        return obj
    try:
        return functools.reduce(getattr, path.split("."), obj)
    except AttributeError:
        if default:
            return default[0]
        raise


def rsetattr(obj, path: str, value) -> None:
    head, _, tail = path.rpartition(".")
    setattr(rgetattr(obj, head), tail, value)


def rhasattr(obj, path: str) -> bool:
    if path == "":
        return True
    for name in path.split("."):
        if not hasattr(obj, name):
            return False
        obj = getattr(obj, name)
    return True


def mixed_precision_dtype(name: str) -> torch.dtype:
    """``--mixed_precision`` value -> dtype (reference hybrid_parallel_config.py ``mixed_precision_dtype``)."""
    return {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}[name]


def print_param_num(model) -> int:
    """Total and trainable parameter counts of this rank's part of the model (reference utils/memory_utils.py)."""
    total = sum(p.numel() for p in model.parameters())
    trainable = sum(p.numel() for p in model.parameters() if p.requires_grad)
    print("Total number of paramerters in networks is {}  ({} trainable)".format(total, trainable))
    return total
