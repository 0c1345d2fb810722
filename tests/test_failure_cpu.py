"""Failure detection on CPU ranks: the failure is made on the host (a rank raises, exits between steps, or stops
beating); the survivors must learn of it from the store before their next collective and leave with RankFailure."""
import json
import os
import subprocess
import sys

import pytest

from dist_utils import ROOT, free_port
from hetu_galvatron_b200.core.failure import Heartbeat, RankFailure

WORKER = os.path.join(ROOT, "tests", "failure_worker.py")


def run(spec, world=3, timeout=90):
    port = free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), OMP_NUM_THREADS="1")
        procs.append(subprocess.Popen([sys.executable, WORKER, json.dumps(spec)], env=env, cwd=ROOT, stdout=subprocess.PIPE,
                                      stderr=subprocess.PIPE, text=True))
    out = {}
    for r, p in enumerate(procs):
        try:
            so, se = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            raise AssertionError("rank %d did not finish" % r)
        for line in so.splitlines():
            if line.startswith("RESULT "):
                out[r] = json.loads(line[7:])
    return out


@pytest.mark.parametrize("mode", ["raise", "exit", "stall"])
def test_survivors_detect_a_host_side_failure(mode):
    res = run({"victim": 1, "mode": mode, "fail_at": 2, "steps": 8, "timeout_s": 1.5, "stall_s": 8})
    for r in (0, 2):
        assert r in res, res
        assert res[r]["detected"] is not None and "1" in res[r]["detected"], res
        assert res[r]["steps"] >= 2
    if mode == "raise":
        assert res[1]["raised"] == "injected host failure"
        assert "injected host failure" in res[0]["detected"]["1"]
    else:
        assert "no heartbeat" in res[0]["detected"]["1"]


def test_clean_run_reports_nothing():
    res = run({"victim": -1, "mode": "none", "steps": 4})
    assert all(v["detected"] is None and v["steps"] == 4 for v in res.values()) and len(res) == 3


def test_heartbeat_with_in_process_store():
    import torch.distributed as dist
    store = dist.HashStore()
    a = Heartbeat(store, 0, 2, interval_s=0.05, timeout_s=0.4).start()
    b = Heartbeat(store, 1, 2, interval_s=0.05, timeout_s=0.4).start()
    assert a.failed_ranks() == {} and b.failed_ranks() == {}
    b.stop(leaving=True)                         # a rank that leaves on purpose is not a failure
    import time
    time.sleep(0.6)
    assert a.failed_ranks() == {}
    c = Heartbeat(store, 1, 2, prefix="other")
    c.report_failure("checkpoint shard unreadable")
    d = Heartbeat(store, 0, 2, prefix="other")
    with pytest.raises(RankFailure, match="checkpoint shard unreadable"):
        d.check()
    a.stop()
