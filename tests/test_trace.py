"""Span recorder and chrome-trace output."""
import json

import torch

from hetu_galvatron_b200.core.hybrid_model import construct_hybrid_parallel_model
from hetu_galvatron_b200.core.plan import HybridPlan
from hetu_galvatron_b200.models import build_model_specs, synthetic_batch
from hetu_galvatron_b200.utils import trace


def test_blocks_and_optimizer_are_traced(tmp_path):
    tr = trace.enable_tracing(0)
    try:
        cfg, specs = build_model_specs("llama", dtype=torch.float32, hidden_size=32, num_heads=2, num_kv_heads=2,
                                       ffn_hidden_size=64, num_layers=2, vocab_size=64, seq_length=16)
        plan = HybridPlan.from_global(2, 1, global_bsz=2, chunks=1)
        model = construct_hybrid_parallel_model(cfg, plan, specs, torch.device("cpu"))
        batch = synthetic_batch("llama", cfg, 2, seed=0, device="cpu")
        with tr.span("iteration", "step"):
            model.forward_backward(batch, 0)
            model.optimizer_step(1e-3)
        out = tr.dump(str(tmp_path / "t"))
        data = json.load(open(out))
        names = {e["name"] for e in data["traceEvents"]}
        assert {"fwd:model_layers_0", "bwd:model_layers_1", "optimizer_step", "iteration", "fwd:lm_head"} <= names
        assert all(e["ph"] == "X" and e["dur"] >= 0 for e in data["traceEvents"])
        assert data["summary"]["fwd:model_layers_0"]["count"] == 1
    finally:
        trace._TRACER = trace.Tracer(False)


def test_disabled_tracer_records_nothing():
    t = trace.Tracer(False)
    with t.span("x"):
        pass
    assert t.dump("/nonexistent/never") is None and t._spans == []
