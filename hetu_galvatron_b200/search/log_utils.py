"""One plain-text log file per search task.

A search task is one point of the outer loops (batch size, micro-batch count, tensor-parallel range, vocab sequence
parallelism, embedding ZeRO-3). Its messages go to ``<log_dir>/search_bsz{B}_chunk{C}/min_tp{a}_max_tp{b}_vsp{v}_embed_sdp{e}.log``
-- the layout of the reference's search logs (galvatron/core/search_engine/utils.py:4-31), so tools that read one read the
other -- through a ``logging.Logger`` that belongs to that task alone: tasks may run on a thread pool without interleaving.
"""
from __future__ import annotations

import logging
import os
from typing import NamedTuple


class SearchTask(NamedTuple):
    bsz: int
    chunk: int
    min_tp: int
    max_tp: int
    vsp: int
    embed_sdp: int

    @property
    def folder(self) -> str:
        return "search_bsz%s_chunk%s" % (self.bsz, self.chunk)

    @property
    def stem(self) -> str:
        return "min_tp%s_max_tp%s_vsp%s_embed_sdp%s" % (self.min_tp, self.max_tp, self.vsp, self.embed_sdp)

    @property
    def logger_name(self) -> str:
        return "galvatron_bsz%s_chunk%s_%s" % (self.bsz, self.chunk, self.stem)


def ensure_log_dir(log_dir: str = "logs") -> str:
    os.makedirs(log_dir, exist_ok=True)
    return log_dir


def task_logger(task: SearchTask, log_dir: str = "logs") -> logging.Logger:
    """The task's logger, created on first use (message text only, file truncated, nothing passed up to the root logger)."""
    log = logging.getLogger(task.logger_name)
    if not log.handlers:
        target = os.path.join(ensure_log_dir(os.path.join(log_dir, task.folder)), task.stem + ".log")
        sink = logging.FileHandler(target, mode="w")
        sink.setFormatter(logging.Formatter("%(message)s"))
        log.addHandler(sink)
        log.setLevel(logging.INFO)
        log.propagate = False
    return log


def get_thread_logger(bsz, chunk, min_tp, max_tp, vsp, embed_sdp, log_dir: str = "logs") -> logging.Logger:
    """``task_logger`` under the reference's name and argument order."""
    return task_logger(SearchTask(bsz, chunk, min_tp, max_tp, vsp, embed_sdp), log_dir)
