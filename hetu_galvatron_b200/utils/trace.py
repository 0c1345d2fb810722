"""Device-timed spans and chrome-trace output (``--trace PATH``).

The reference's only per-iteration instrumentation is the runtime profiler's pair of CUDA events around an iteration
(galvatron/core/profiler/runtime_profiler.py:189-250); torch.profiler is used only by its hardware micro-benchmarks.
Here every block's forward and backward, the optimizer step and user-named regions are bracketed by CUDA events on
the launching stream (no host synchronisation while recording); ``dump`` resolves them once and writes a
``chrome://tracing`` / Perfetto JSON per rank plus a per-name summary (count, total ms, mean ms)."""
from __future__ import annotations

import json
import time
from collections import defaultdict
from contextlib import contextmanager
from typing import Dict, List, Optional

import torch


class Tracer:
    def __init__(self, enabled: bool = False, rank: int = 0, max_spans: int = 200000):
        self.enabled, self.rank, self.max_spans = enabled, rank, max_spans
        self._spans: List[tuple] = []
        self._open: Dict[str, object] = {}
        self._cuda = torch.cuda.is_available()
        self._base = None

    def _mark(self):
        if self._cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            if self._base is None:
                self._base = ev
            return ev
        t = time.perf_counter()
        if self._base is None:
            self._base = t
        return t

    def begin(self, name: str, cat: str = "compute") -> None:
        if self.enabled and len(self._spans) < self.max_spans:
            self._open[name] = (self._mark(), cat)

    def end(self, name: str) -> None:
        if self.enabled and name in self._open:
            start, cat = self._open.pop(name)
            self._spans.append((name, cat, start, self._mark()))

    @contextmanager
    def span(self, name: str, cat: str = "compute"):
        if not self.enabled:
            yield
            return
        self.begin(name, cat)
        try:
            yield
        finally:
            self.end(name)

    def _resolve(self):
        if self._cuda:
            torch.cuda.synchronize()
            return [(n, c, self._base.elapsed_time(a) * 1e3, a.elapsed_time(b) * 1e3) for n, c, a, b in self._spans]
        return [(n, c, (a - self._base) * 1e6, (b - a) * 1e6) for n, c, a, b in self._spans]

    def summary(self) -> Dict[str, dict]:
        agg = defaultdict(lambda: [0, 0.0])
        for n, _, _, dur in self._resolve():
            agg[n][0] += 1
            agg[n][1] += dur / 1e3
        return {n: {"count": c, "total_ms": round(t, 4), "mean_ms": round(t / c, 4)} for n, (c, t) in agg.items()}

    def dump(self, path: str) -> Optional[str]:
        if not self.enabled:
            return None
        events = [{"name": n, "cat": c, "ph": "X", "ts": ts, "dur": dur, "pid": self.rank, "tid": c}
                  for n, c, ts, dur in self._resolve()]
        out = path if path.endswith(".json") else "%s_rank%d.json" % (path, self.rank)
        with open(out, "w") as fp:
            json.dump({"traceEvents": events, "displayTimeUnit": "ms", "summary": self.summary()}, fp)
        return out

    def clear(self) -> None:
        self._spans, self._open, self._base = [], {}, None


_TRACER = Tracer(False)


def get_tracer() -> Tracer:
    return _TRACER


def enable_tracing(rank: int = 0) -> Tracer:
    global _TRACER
    _TRACER = Tracer(True, rank)
    return _TRACER
