"""Failure detection for multi-rank jobs: host heartbeats, device error words, a common exit, and re-planning.

The reference has none of this beyond the process-group timeout (megatron/training/arguments.py:1341
``--distributed-timeout-minutes``; tests fail a run when a rank subprocess exits non-zero, tests/conftest.py:61-69).
Here:

* ``Heartbeat``: every rank bumps a counter in the job's key-value store from a daemon thread; ``check()`` (called by
  the training loop between steps, i.e. with none of this rank's kernels or collectives in flight) raises
  ``RankFailure`` naming the ranks whose counter stopped for longer than ``timeout_s`` or that published a failure.
  A rank that fails on the host publishes its reason with ``report_failure`` before it leaves, so the others learn
  of it before their next collective instead of at the process-group timeout.
* ``check_kernel_errors``: reads the error word that this package's bounded device waits write when they give up
  (csrc/include/gv_ptx.cuh, gv_comm.cuh), publishes it and raises on every rank of the job.
* ``replan_for_world_size``: after a rank loss, searches the best plan for the surviving world size from the same
  profiles (the search is CPU-only), for a restart from the last checkpoint.

Nothing here faults, traps or hangs a GPU; the failures these paths handle are made on the host in the tests
(a rank that raises or exits, a store key that is never written, a device wait on a flag nothing sets).
"""
from __future__ import annotations

import threading
import time
from typing import Dict, List, Optional

import torch.distributed as dist


class RankFailure(RuntimeError):
    def __init__(self, failed: Dict[int, str]):
        self.failed = dict(failed)
        super().__init__("rank failure detected: " + "; ".join("rank %d: %s" % kv for kv in sorted(self.failed.items())))


class Heartbeat:
    """Liveness over a ``torch.distributed`` key-value store (TCPStore / FileStore / HashStore)."""

    def __init__(self, store, rank: int, world_size: int, interval_s: float = 0.5, timeout_s: float = 10.0, prefix: str = "gv_hb"):
        self.store, self.rank, self.world = store, rank, world_size
        self.interval, self.timeout, self.prefix = interval_s, timeout_s, prefix
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._seen: Dict[int, tuple] = {}          # rank -> (last counter value, local time it changed)
        self._beats = 0

    def _key(self, kind: str, rank: int) -> str:
        return "%s/%s/%d" % (self.prefix, kind, rank)

    def start(self) -> "Heartbeat":
        self.store.set(self._key("beat", self.rank), "0")
        self._thread = threading.Thread(target=self._run, name="gv-heartbeat", daemon=True)
        self._thread.start()
        return self

    def _run(self) -> None:
        while not self._stop.wait(self.interval):
            self._beats += 1
            try:
                self.store.set(self._key("beat", self.rank), str(self._beats))
            except Exception:
                return                              # the store is gone: the job is being torn down

    def stop(self, leaving: bool = True) -> None:
        """``leaving``: tell the peers that this rank left on purpose (they stop expecting its beats)."""
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1)
        if leaving:
            try:
                self.store.set(self._key("left", self.rank), "1")
            except Exception:
                pass

    def report_failure(self, reason: str) -> None:
        self.store.set(self._key("fail", self.rank), reason[:500])

    def _get(self, key: str) -> Optional[str]:
        try:
            if hasattr(self.store, "check") and not self.store.check([key]):
                return None
            return self.store.get(key).decode()
        except Exception:
            return None

    def failed_ranks(self) -> Dict[int, str]:
        now = time.monotonic()
        bad: Dict[int, str] = {}
        for r in range(self.world):
            if r == self.rank:
                continue
            why = self._get(self._key("fail", r))
            if why is not None:
                bad[r] = why
                continue
            if self._get(self._key("left", r)) is not None:
                continue
            beat = self._get(self._key("beat", r))
            last = self._seen.get(r)
            if last is None or beat != last[0]:
                self._seen[r] = (beat, now)
            elif now - last[1] > self.timeout:
                bad[r] = "no heartbeat for %.1f s" % (now - last[1])
        return bad

    def check(self) -> None:
        bad = self.failed_ranks()
        if bad:
            raise RankFailure(bad)

    def wait_for_failure(self, max_wait_s: float) -> Dict[int, str]:
        """Poll until a peer is seen failed or ``max_wait_s`` passes (used where a rank has nothing else to do)."""
        end = time.monotonic() + max_wait_s
        while time.monotonic() < end:
            bad = self.failed_ranks()
            if bad:
                return bad
            time.sleep(min(self.interval, 0.2))
        return {}


def check_kernel_errors(heartbeat: Optional[Heartbeat] = None) -> None:
    """Raise if a bounded device wait of this process gave up; publish it so the other ranks stop too."""
    from ..ops import _lib

    err = _lib.read_error()
    if err is None:
        return
    msg = "device wait gave up at site 0x%x (code 0x%x, aux %d / %d)" % (err["site"], err["code"], err["aux0"], err["aux1"])
    if heartbeat is not None:
        heartbeat.report_failure(msg)
    raise RankFailure({heartbeat.rank if heartbeat is not None else (dist.get_rank() if dist.is_initialized() else 0): msg})


def guarded_step(step_fn, heartbeat: Heartbeat, check_device: bool = True, grace_s: Optional[float] = None):
    """Run one training step between two health checks.

    An exception inside the step is either this rank's own failure or the echo of a peer's (a collective that ended
    with an error because the peer is gone). A peer failure already visible in the store wins; a runtime error gets
    ``grace_s`` (default 2 x the heartbeat timeout) for such evidence to appear; otherwise the exception is published
    as this rank's failure and re-raised."""
    heartbeat.check()
    try:
        out = step_fn()
    except RankFailure:
        raise
    except BaseException as exc:
        bad = heartbeat.failed_ranks()
        if not bad and isinstance(exc, RuntimeError):
            bad = heartbeat.wait_for_failure(2 * heartbeat.timeout if grace_s is None else grace_s)
        if bad:
            raise RankFailure(bad) from exc
        heartbeat.report_failure("%s: %s" % (type(exc).__name__, exc))
        raise
    if check_device:
        check_kernel_errors(heartbeat)
    return out


def replan_for_world_size(search_args, program_path: str, layer_configs: List[dict], model_name: str, world_size: int):
    """Best plan for ``world_size`` GPUs from the profiles under ``program_path/configs`` (after a rank loss the job
    restarts from its last checkpoint's weights, converted with the g2h / h2g tools, under this plan)."""
    from ..search import GalvatronSearchEngine

    nodes = max(1, world_size // max(1, search_args.num_gpus_per_node))
    search_args.num_nodes = nodes
    search_args.num_gpus_per_node = world_size // nodes
    engine = GalvatronSearchEngine(search_args)
    engine.set_search_engine_info(program_path, layer_configs, model_name)
    engine.initialize_search_engine()
    return engine.parallelism_optimization()
