import json
import os
import socket
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "dist_worker.py")


def free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def run_worker(spec: dict, world: int, timeout: int = 600, worker: str = WORKER):
    env = dict(os.environ)
    env["OMP_NUM_THREADS"] = "1"
    env.setdefault("NCCL_NVLS_ENABLE", "0")
    for attempt in range(3):
        if world == 1:
            cmd = [sys.executable, worker, json.dumps(spec)]
        else:
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
                   "--master-addr", "127.0.0.1", "--master-port", str(free_port()), worker, json.dumps(spec)]
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)
        if r.returncode == 0 or "EADDRINUSE" not in r.stderr:
            break           # only a lost race for the rendezvous port is worth another try
    if r.returncode != 0:
        raise RuntimeError("worker failed:\n" + r.stdout[-3000:] + "\n" + r.stderr[-6000:])
    for line in r.stdout.splitlines():
        if line.startswith("LOSSES "):
            return json.loads(line[len("LOSSES "):])
    raise RuntimeError("worker printed no losses:\n" + r.stdout[-2000:] + r.stderr[-2000:])
