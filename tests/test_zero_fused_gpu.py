"""The data-parallel engine on this package's own peer-memory kernels (``impl="fused"``: gradient reduce-scatter,
AdamW + parameter push, ZeRO-3 pull gathers) against the same engine on NCCL, on 2 GPUs: DDP / ZeRO-2 / ZeRO-3, one
reduction per step or per micro-batch, with and without gradient clipping (reference behaviour:
galvatron/core/runtime/pipeline/sp_grad_reduce.py:93-132, galvatron/core/runtime/parallel.py:116-138,202-213)."""
import json
import os
import subprocess
import sys

import pytest

from dist_utils import ROOT, free_port

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

MODEL = dict(hidden_size=256, num_heads=4, num_kv_heads=2, ffn_hidden_size=512, num_layers=4, vocab_size=1024, seq_length=128)
CASES = [dict(dp=dp, chunks=2, clip=clip, **{"async": a}) for dp in ("ddp", "zero2", "zero3") for a in (True, False) for clip in (1.0, 0.0)]
CASES += [dict(dp="zero2", chunks=2, clip=1.0, bf16_grads=True, **{"async": True}),
          dict(dp="zero3", chunks=2, clip=1.0, ckpt=1, bf16_grads=True, **{"async": True})]


def test_fused_zero_engine_matches_nccl_engine():
    spec = {"model": MODEL, "global_bsz": 8, "steps": 4, "cases": CASES, "profile_case": len(CASES) - 2}
    env = dict(os.environ, OMP_NUM_THREADS="1")
    env.setdefault("NCCL_NVLS_ENABLE", "0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(free_port()), os.path.join(ROOT, "tests", "zero_fused_worker.py"), json.dumps(spec)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=1200, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-6000:]
    line = [ln for ln in r.stdout.splitlines() if ln.startswith("RESULT ")][-1]
    results = json.loads(line[len("RESULT "):])
    out_dir = os.environ.get("GV_TEST_RESULTS_DIR", "")      # where to keep the measured figures, if anywhere
    if out_dir and os.path.isdir(out_dir):
        json.dump(results, open(os.path.join(out_dir, "zero_fused_vs_nccl.json"), "w"), indent=1)
    for res in results:
        assert res["impl"] == "fused" and res["impl_ref"] == "nccl", res
        assert res["kernel_error"] is None, res
        assert res["loss_diff"] < 3e-2, res
        assert res["param_rel_diff"] < 2e-3, res
    prof = results[spec["profile_case"]]
    # with the fused engine a ZeRO-2 step launches no NCCL reduce-scatter / all-gather kernel: what is left on NCCL is
    # the scalar all-reduce of the gradient norm (and of the reported loss)
    assert prof["own_comm_kernels"], prof
    assert not [k for k in prof["nccl_kernels"] if "ReduceScatter" in k or "AllGather" in k], prof["nccl_kernels"]
