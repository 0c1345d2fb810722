"""Zigzag ring attention on 2 GPUs (bf16, native attention kernels, log-sum-exp merge kernel) against fp32 attention
over the whole sequence: blocks as NCCL point-to-point messages and as pulls from peer memory."""
import json
import os

import pytest

from dist_utils import ROOT, run_worker

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

CASES = [dict(s=512, b=2, hq=4, hk=2, dh=128, causal=True), dict(s=1024, b=1, hq=2, hk=2, dh=64, causal=False)]


@pytest.mark.parametrize("impl", ["nccl", "fused"])
def test_ring_attention_gpu_matches_whole_sequence(impl):
    import subprocess
    import sys
    from dist_utils import free_port
    env = dict(os.environ, OMP_NUM_THREADS="1")
    env.setdefault("NCCL_NVLS_ENABLE", "0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(free_port()), os.path.join(ROOT, "tests", "ring_worker.py"),
           json.dumps({"cases": CASES, "device": "cuda", "impl": impl})]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    worst = float([ln for ln in r.stdout.splitlines() if ln.startswith("WORST")][-1].split()[1])
    assert worst < 3e-2, worst
