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


def _spawn_ranks(cmd_tail, world: int, env: dict, timeout: int):
    """Start ``world`` ranks directly (RANK / LOCAL_RANK / WORLD_SIZE / MASTER_* in the environment, as the reference's
    tests/conftest.py:31-71 does) and wait for them; when one rank fails the others are stopped by their own PIDs."""
    import tempfile
    import time

    port = str(free_port())
    procs, files = [], []
    for rank in range(world):
        e = dict(env, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=port)
        out, err = tempfile.TemporaryFile(mode="w+"), tempfile.TemporaryFile(mode="w+")
        files.append((out, err))
        procs.append(subprocess.Popen([sys.executable] + cmd_tail, stdout=out, stderr=err, env=e, cwd=ROOT))
    deadline = time.time() + timeout
    failed = False
    while True:
        codes = [p.poll() for p in procs]
        if all(c is not None for c in codes):
            break
        if any(c not in (None, 0) for c in codes) or time.time() > deadline:
            failed = True
            time.sleep(1.0)                       # let the failing rank's neighbours print their own errors
            for p in procs:
                if p.poll() is None:
                    p.kill()
            for p in procs:
                p.wait()
            break
        time.sleep(0.05)
    texts = []
    for out, err in files:
        out.seek(0), err.seek(0)
        texts.append((out.read(), err.read()))
        out.close(), err.close()
    rc = 1 if failed else max(p.returncode for p in procs)
    # the last rank prints the result line; the first failing rank's stderr is the useful one
    stdout = "".join(t[0] for t in texts)
    bad = [t[1] for p, t in zip(procs, texts) if p.returncode not in (0, None, -9)] or [t[1] for t in texts]
    return rc, stdout, "\n".join(bad)


def run_worker(spec: dict, world: int, timeout: int = 600, worker: str = WORKER):
    env = dict(os.environ)
    env["OMP_NUM_THREADS"] = "1"
    env.setdefault("NCCL_NVLS_ENABLE", "0")
    for attempt in range(3):
        if world == 1:
            r = subprocess.run([sys.executable, worker, json.dumps(spec)], capture_output=True, text=True, timeout=timeout,
                               env=env, cwd=ROOT)
            rc, out, err = r.returncode, r.stdout, r.stderr
        elif spec.get("device", "cpu") == "cuda" or worker != WORKER:
            # GPU ranks go through the launcher the benchmark and the training scripts use
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
                   "--master-addr", "127.0.0.1", "--master-port", str(free_port()), worker, json.dumps(spec)]
            r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)
            rc, out, err = r.returncode, r.stdout, r.stderr
        else:
            rc, out, err = _spawn_ranks([worker, json.dumps(spec)], world, env, timeout)
        if rc == 0 or "EADDRINUSE" not in err:
            break           # only a lost race for the rendezvous port is worth another try
    if rc != 0:
        raise RuntimeError("worker failed:\n" + out[-3000:] + "\n" + err[-6000:])
    losses = skipped = None
    for line in out.splitlines():
        if line.startswith("LOSSES "):
            losses = json.loads(line[len("LOSSES "):])
        if line.startswith("SKIPPED "):
            skipped = json.loads(line[len("SKIPPED "):])
    if losses is None:
        raise RuntimeError("worker printed no losses:\n" + out[-2000:] + err[-2000:])
    if spec.get("report_skipped"):
        return losses, skipped          # per rank: which optimizer steps were skipped for a non-finite gradient norm
    return losses
