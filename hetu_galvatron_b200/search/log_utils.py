"""One log file per search task (reference: galvatron/core/search_engine/utils.py:4-31)."""
from __future__ import annotations

import logging
import os


def ensure_log_dir(log_dir: str = "logs") -> str:
    os.makedirs(log_dir, exist_ok=True)
    return log_dir


def get_thread_logger(bsz, chunk, min_tp, max_tp, vsp, embed_sdp, log_dir: str = "logs") -> logging.Logger:
    name = f"galvatron_bsz{bsz}_chunk{chunk}_min_tp{min_tp}_max_tp{max_tp}_vsp{vsp}_embed_sdp{embed_sdp}"
    logger = logging.getLogger(name)
    if logger.handlers:
        return logger
    logger.setLevel(logging.INFO)
    sub = os.path.join(log_dir, f"search_bsz{bsz}_chunk{chunk}")
    os.makedirs(sub, exist_ok=True)
    handler = logging.FileHandler(os.path.join(sub, f"min_tp{min_tp}_max_tp{max_tp}_vsp{vsp}_embed_sdp{embed_sdp}.log"), mode="w")
    handler.setFormatter(logging.Formatter("%(message)s"))
    logger.addHandler(handler)
    logger.propagate = False
    return logger
