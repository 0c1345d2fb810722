"""Recovery after a rank loss, end to end on CPU ranks: a 4-rank job saves a checkpoint with portable optimizer state;
the search is re-run for the surviving world size (``replan_for_world_size``); the job resumes on 2 ranks under the new
plan and continues with the losses of the uninterrupted run. The loss of ranks is decided on the host; detecting it is
covered by test_failure_cpu.py."""
import json

from dist_utils import run_worker
from hetu_galvatron_b200.core.failure import replan_for_world_size
from hetu_galvatron_b200.core.plan import HybridPlan
from search_utils import search_args, write_tiny_gpt_profiles

MODEL = dict(hidden_size=256, num_heads=4, ffn_hidden_size=1024, num_layers=4, vocab_size=1024, seq_length=128)
LAYERS = [{"hidden_size": 256, "layer_num": 4, "seq_len": 128}]


def test_replan_for_the_surviving_ranks_and_resume(tmp_path):
    cfg_dir, hw_dir, name = write_tiny_gpt_profiles(str(tmp_path / "prof"), worlds=(4, 2))

    def args_for(world):
        return search_args(num_gpus_per_node=world, memory_constraint=8, settle_bsz=8, settle_chunk=1, mixed_precision="fp32",
                           max_tp_deg=world, max_pp_deg=world, time_profiling_path=cfg_dir, memory_profiling_path=cfg_dir,
                           allreduce_bandwidth_config_path=hw_dir, p2p_bandwidth_config_path=hw_dir, overlap_coe_path=hw_dir,
                           sp_time_path=hw_dir, output_config_path=str(tmp_path / "plans"), log_dir=str(tmp_path / "logs"),
                           hidden_size=256, default_dp_type="zero2")

    # the job as planned for 4 ranks
    a4 = args_for(4)
    thr4 = replan_for_world_size(a4, str(tmp_path / "prof"), LAYERS, name, 4)
    plan4 = str(tmp_path / "plans" / ("galvatron_config_%s_1nodes_4gpus_per_node_8GB_fp32_bsz8.json" % name))
    p4 = HybridPlan.from_json(plan4, 4)
    p4.validate(4, 4)
    steps, ck = 6, str(tmp_path / "ck")
    full = run_worker({"family": "gpt", "model": MODEL, "plan_json": plan4, "steps": steps, "seed": 0,
                       "save": {"dir": ck, "iter": 3, "portable": True}}, 4)
    assert len(full) == steps

    # two ranks are lost after iteration 3: plan again for the two survivors and resume from the checkpoint
    thr2 = replan_for_world_size(args_for(4), str(tmp_path / "prof"), LAYERS, name, 2)
    plan2 = str(tmp_path / "plans" / ("galvatron_config_%s_1nodes_2gpus_per_node_8GB_fp32_bsz8.json" % name))
    p2 = HybridPlan.from_json(plan2, 4)
    p2.validate(2, 4)
    assert 0 < thr2 < thr4                                        # half the ranks, less throughput
    assert p2.tp_sizes_enc == p4.tp_sizes_enc                     # the checkpoint's file layout (per tensor-parallel rank) still fits
    resumed = run_worker({"family": "gpt", "model": MODEL, "plan_json": plan2, "steps": steps, "seed": 0,
                          "load": {"dir": ck, "iter": 3, "allow_plan_change": True}}, 2)
    assert len(resumed) == steps - 3
    for a, b in zip(resumed, full[3:]):
        assert abs(a - b) < 2e-4 * max(1.0, abs(b)), (resumed, full)
    assert json.load(open(plan2))["global_bsz"] == 8
