"""HybridPlan: GLOBAL flags and strategy JSON give the same per-layer lists; default micro-batch count; validity checks
(reference: galvatron/core/runtime/hybrid_parallel_config.py:17-158 flags / JSON, :190-217 checks, :351-361 chunks)."""
import json

import pytest

from hetu_galvatron_b200.core.plan import HybridPlan, even_pp_division


def test_global_flags_expand_to_per_layer_lists():
    p = HybridPlan.from_global(8, 8, pp_deg=2, global_tp_deg=2, sdp=1, global_checkpoint=1, vocab_tp=2, chunks=4,
                               global_bsz=16, default_dp_type="zero2", sequence_parallel=True)
    assert p.tp_sizes_enc == [2] * 8 and p.dp_types_enc == [1] * 8 and p.checkpoint_flags_enc == [1] * 8
    assert p.use_sp == [0] * 8 and p.cp_sizes_enc == [1] * 8 and p.pp_division == [4, 4]
    assert p.pp_ranks_enc == [0] * 4 + [1] * 4 and p.num_layers == 8
    assert p.layer_dp_type(0) == "zero3"
    p.validate(8, num_heads=4)
    u = HybridPlan.from_global(4, 8, pp_deg=1, global_tp_deg=4, use_ulysses=True, global_bsz=8)
    assert u.use_sp == [1] * 4 and u.vocab_sp == 1 and u.layer_dp_type(2) == "ddp"
    u.validate(8, num_heads=8)
    with pytest.raises(AssertionError, match="Ulysses"):
        u.validate(8, num_heads=6)


def test_default_micro_batch_count():
    # chunks = -1: one micro-batch without a pipeline, ceil(local batch / 4) with one
    assert HybridPlan.from_global(8, 8, pp_deg=1, chunks=-1, global_bsz=64).chunks == 1
    assert HybridPlan.from_global(8, 8, pp_deg=2, chunks=-1, global_bsz=64).chunks == 4          # local 16 -> 4
    assert HybridPlan.from_global(8, 8, pp_deg=2, global_tp_deg=2, vocab_tp=2, chunks=-1, global_bsz=72).chunks == 9
    assert HybridPlan.from_global(8, 8, pp_deg=4, chunks=-1, global_bsz=2).chunks == 1
    assert even_pp_division(10, 4) == [2, 2, 2, 4] and even_pp_division(8, 1) == [8]


def test_json_round_trip_and_defaults(tmp_path):
    p = HybridPlan.from_global(6, 8, pp_deg=2, global_tp_deg=2, global_cp_deg=2, vocab_tp=2, vocab_cp=2, chunks=2, global_bsz=8,
                               pipeline_type="gpipe", default_dp_type="zero2", embed_sdp=1, pp_division=[2, 4])
    p.tp_sizes_enc[0], p.dp_types_enc[1], p.use_sp[2], p.checkpoint_flags_enc[3] = 4, 1, 1, 1
    p.cp_sizes_enc[0] = 1
    path = tmp_path / "plan.json"
    path.write_text(json.dumps(p.to_json()))
    q = HybridPlan.from_json(str(path), 6)
    for f in ("pp_deg", "tp_sizes_enc", "cp_sizes_enc", "dp_types_enc", "use_sp", "checkpoint_flags_enc", "pp_division",
              "global_bsz", "chunks", "pipeline_type", "default_dp_type", "vocab_tp", "vocab_sp", "vocab_cp", "embed_sdp"):
        assert getattr(p, f) == getattr(q, f), f
    assert q.as_runtime_dict()["pp_ranks_enc"] == [0, 0, 1, 1, 1, 1]
    # keys the reference's own search never writes are optional
    minimal = {"pp_deg": 1, "tp_sizes_enc": "1,2", "tp_consecutive_flags": "1,1", "dp_types_enc": "0,1", "global_bsz": 8, "chunks": 1}
    m = HybridPlan.from_json(minimal, 2, sequence_parallel=True)
    assert m.cp_sizes_enc == [1, 1] and m.use_sp == [0, 0] and m.checkpoint_flags_enc == [0, 0] and m.pp_division == [2]
    assert m.vocab_cp == 1 and m.sequence_parallel is True
    with pytest.raises(ValueError, match="does not match"):
        HybridPlan.from_json(minimal, 3)
    assert "tp_sizes_enc: 1,2" in m.describe() and "Galvatron Parallel Config" in m.describe()


@pytest.mark.parametrize("change,message", [
    (dict(global_bsz=7, chunks=1), "multiple of world_size"),
    (dict(chunks=3), "micro-batches"),
    (dict(pp_division=[3, 4]), "pp_division"),
    (dict(tp_sizes_enc=[3] * 8), "tp\\*cp must divide|powers of two"),
    (dict(tp_sizes_enc=[8] * 8), "tp\\*cp must divide"),
    (dict(pipeline_type="interleaved"), None),
    (dict(use_sp=[0] * 7), "one entry per layer"),
])
def test_invalid_plans_are_rejected(change, message):
    p = HybridPlan.from_global(8, 8, pp_deg=2, global_tp_deg=2, vocab_tp=2, chunks=2, global_bsz=8)
    p.validate(8)
    for k, v in change.items():
        setattr(p, k, v)
    with pytest.raises(AssertionError, match=message):
        p.validate(8)


def test_grouped_query_models_limit_the_tensor_parallel_degree():
    p = HybridPlan.from_global(4, 8, global_tp_deg=4, vocab_tp=4, global_bsz=8)
    p.validate(8, num_heads=8, num_kv_heads=4)
    with pytest.raises(AssertionError, match="KV-head count"):
        p.validate(8, num_heads=8, num_kv_heads=2)
    u = HybridPlan.from_global(4, 8, global_tp_deg=4, use_ulysses=True, global_bsz=8)
    u.validate(8, num_heads=8, num_kv_heads=2)          # Ulysses keeps whole weights: no such limit
