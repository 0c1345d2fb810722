"""Memory reporting helpers (reference: galvatron/utils/memory_utils.py; galvatron/core/profiler/utils.py:8-19)."""
from __future__ import annotations

import torch


def memory_stats_mb(device=None) -> dict:
    if not torch.cuda.is_available():
        return {"allocated": 0.0, "max_allocated": 0.0, "reserved": 0.0, "max_reserved": 0.0}
    mb = 2 ** 20
    return {
        "allocated": torch.cuda.memory_allocated(device) / mb,
        "max_allocated": torch.cuda.max_memory_allocated(device) / mb,
        "reserved": torch.cuda.memory_reserved(device) / mb,
        "max_reserved": torch.cuda.max_memory_reserved(device) / mb,
    }


def print_peak_memory(prefix: str, device, profile_type: str = "allocated") -> tuple:
    s = memory_stats_mb(device)
    if profile_type == "allocated":
        cur, peak = s["allocated"], s["max_allocated"]
    else:
        cur, peak = s["reserved"], s["max_reserved"]
    print("%s: current %.2f MB, peak %.2f MB (%s)" % (prefix, cur, peak, profile_type), flush=True)
    return peak, cur
