"""Worker of tests/test_failure_cpu.py: gloo ranks with heartbeats; one rank fails on the host in a chosen way."""
import json
import os
import sys
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from hetu_galvatron_b200.core.failure import Heartbeat, RankFailure, guarded_step  # noqa: E402


def main():
    spec = json.loads(sys.argv[1])
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    store = dist.TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]) + 1, world, is_master=(rank == 0), timeout=__import__("datetime").timedelta(seconds=30))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    hb = Heartbeat(store, rank, world, interval_s=0.1, timeout_s=spec.get("timeout_s", 1.5)).start()
    victim, mode, fail_at = spec["victim"], spec["mode"], spec.get("fail_at", 2)
    x = torch.ones(4)
    result = {"rank": rank, "steps": 0, "detected": None}

    def step():
        if rank == victim and result["steps"] == fail_at:
            if mode == "raise":
                raise ValueError("injected host failure")
            if mode == "exit":
                os._exit(0)                 # vanishes between steps without a word
            if mode == "stall":
                hb._stop.set()              # heartbeat thread dies, the rank never joins again
                time.sleep(spec.get("stall_s", 6))
                os._exit(0)
        dist.all_reduce(x)
        return float(x[0])

    try:
        for _ in range(spec.get("steps", 6)):
            guarded_step(step, hb, check_device=False)
            result["steps"] += 1
            time.sleep(0.3)                 # host work between steps: where a failure notice can arrive
    except RankFailure as exc:
        result["detected"] = {str(k): v for k, v in exc.failed.items()}
    except ValueError as exc:
        result["raised"] = str(exc)
    print("RESULT " + json.dumps(result), flush=True)
    hb.stop(leaving=result["detected"] is None and "raised" not in result)
    os._exit(0)                             # no collective teardown: peers may be gone


if __name__ == "__main__":
    main()
