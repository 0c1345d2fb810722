"""End-to-end single-GPU model tests: the kernel path against the fp32 CPU path of the same model."""
import pytest
import torch

from hetu_galvatron_b200.core.hybrid_model import construct_hybrid_parallel_model
from hetu_galvatron_b200.core.plan import HybridPlan
from hetu_galvatron_b200.models.llama import llama_specs
from hetu_galvatron_b200.models.transformer import ModelConfig
from hetu_galvatron_b200.ops import _lib

pytestmark = pytest.mark.gpu


def _run(device, dtype, steps=3, ckpt=0):
    cfg = ModelConfig(hidden_size=256, num_heads=4, num_kv_heads=2, ffn_hidden_size=704, num_layers=2, vocab_size=1024,
                      seq_length=128, dtype=dtype)
    plan = HybridPlan.from_global(cfg.num_layers, 1, global_bsz=4, chunks=2, global_checkpoint=ckpt)
    model = construct_hybrid_parallel_model(cfg, plan, llama_specs(cfg), device)
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(0, cfg.vocab_size, (4, cfg.seq_length + 1), generator=g).to(device)
    out = []
    for it in range(steps):
        loss = model.forward_backward((tok[:, :-1], tok[:, 1:]), it)
        model.optimizer_step(1e-3, max_grad_norm=1.0)
        model.zero_grad()
        out.append(float(loss))
    return out


@pytest.mark.parametrize("ckpt", [0, 1])
def test_llama_gpu_matches_cpu_fp32(ckpt):
    gpu = _run(torch.device("cuda"), torch.bfloat16, ckpt=ckpt)
    cpu = _run(torch.device("cpu"), torch.float32, ckpt=ckpt)
    assert _lib.read_error() is None
    for a, b in zip(gpu, cpu):
        assert abs(a - b) < 5e-2, (gpu, cpu)
    assert gpu[-1] < gpu[0]


def test_graft_smoke():
    import __graft_entry__ as g
    g.smoke()
