"""Hybrid-parallel plans on real GPUs over NCCL (bf16, native kernels) against the single-GPU run."""
import pytest

from dist_utils import run_worker

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

MODEL = dict(hidden_size=256, num_heads=4, num_kv_heads=2, ffn_hidden_size=512, num_layers=4, vocab_size=1024, seq_length=128)
_BASE = {}


def baseline():
    if "b" not in _BASE:
        _BASE["b"] = run_worker({"family": "llama", "model": MODEL, "plan": {"global_bsz": 8, "chunks": 1}, "steps": 3,
                                 "device": "cuda", "dtype": "bf16"}, 1)
    return _BASE["b"]


CASES = {
    "dp2_zero2": dict(global_bsz=8, chunks=2, default_dp_type="zero2"),
    "dp2_zero3_ckpt": dict(global_bsz=8, chunks=2, sdp=1, global_checkpoint=1),
    "tp2_sp": dict(global_bsz=8, global_tp_deg=2, vocab_tp=2, sequence_parallel=True),
    "ulysses2": dict(global_bsz=8, global_tp_deg=2, use_ulysses=True, vocab_tp=2),
    "cp2": dict(global_bsz=8, global_cp_deg=2, vocab_cp=2),
    "pp2_1f1b": dict(global_bsz=8, pp_deg=2, chunks=4),
}


@pytest.mark.parametrize("name", list(CASES))
def test_gpu_plan_matches_single_gpu(name):
    spec = {"family": "llama", "model": MODEL, "plan": CASES[name], "steps": 3, "device": "cuda", "dtype": "bf16"}
    losses = run_worker(spec, 2)
    ref = baseline()
    for a, b in zip(losses, ref):
        assert abs(a - b) < 6e-2, (losses, ref)
