"""Every plan JSON shipped under models/<family>_programs/configs loads against the model size its file name carries and
is a valid layout for the GPU count it names; every family directory has the reference's four programs and scripts."""
import glob
import os
import re

import pytest
import torch

from hetu_galvatron_b200.core.plan import HybridPlan
from hetu_galvatron_b200.models import build_model_specs

MODELS = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "hetu_galvatron_b200", "models")
PLANS = sorted(glob.glob(os.path.join(MODELS, "*_programs", "configs", "galvatron_config_*.json")))


def test_plans_are_shipped_for_every_family():
    families = {os.path.basename(os.path.dirname(os.path.dirname(p))) for p in PLANS}
    assert families >= {"llama_programs", "gpt_programs", "bert_programs", "vit_programs", "t5_programs", "swin_programs"}


@pytest.mark.parametrize("path", PLANS, ids=[os.path.basename(p)[len("galvatron_config_"):-5] for p in PLANS])
def test_shipped_plan_fits_its_model(path):
    family = os.path.basename(os.path.dirname(os.path.dirname(path)))[:-len("_programs")]
    searched = re.match(r"galvatron_config_.+_(\d+)nodes_(\d+)gpus_per_node_", os.path.basename(path))
    if searched:          # written by the search engine: named after the profile, not after a model size
        plan = HybridPlan.from_json(path)
        plan.validate(int(searched.group(1)) * int(searched.group(2)))
        assert sum(plan.pp_division) == len(plan.tp_sizes_enc) and plan.global_bsz % plan.chunks == 0
        return
    m = re.match(r"galvatron_config_(.+)_(\d+)gpus_", os.path.basename(path))
    size, world = m.group(1), int(m.group(2))
    with torch.device("meta"):
        cfg, specs = build_model_specs(family, dtype=torch.bfloat16, model_size=size)
    n_layers = len([s for s in specs if s.layer_index is not None])
    plan = HybridPlan.from_json(path, n_layers)
    plan.validate(world, cfg.num_heads)
    assert sum(plan.pp_division) == n_layers and len(plan.pp_division) == plan.pp_deg
    assert plan.global_bsz % plan.chunks == 0 or plan.chunks == 1


@pytest.mark.parametrize("family", ["llama", "gpt", "bert", "vit", "t5", "swin", "llama_fa", "gpt_fa"])
def test_family_directory_has_programs_and_scripts(family):
    d = os.path.join(MODELS, family + "_programs")
    for prog in ("train_dist.py", "train_dist_random.py", "profiler.py", "search_dist.py"):
        assert os.path.exists(os.path.join(d, prog)), prog
    for script in ("train_dist.sh", "train_dist_random.sh", "profile_computation.sh", "profile_memory.sh", "search_dist.sh"):
        path = os.path.join(d, "scripts", script)
        assert os.path.exists(path) and os.access(path, os.X_OK), script


@pytest.mark.parametrize("gpus,measured_gib", [(1, 127.9), (2, 90.2), (8, 62.0)])
def test_shipped_llama_profile_predicts_the_measured_peak_memory(gpus, measured_gib, capsys):
    """Llama-7B, seq 4096, 8 sequences per GPU in 4 micro-batches, ZeRO-2 data parallel with bf16 gradient buffers: peak
    allocated memory measured on B200 against the prediction from the shipped memory profile under the engine layout."""
    from hetu_galvatron_b200.models.runner import search

    table = search("llama", argv=[
        "--model_size", "llama-7b", "--set_seqlen_manually", "1", "--seq_length", "4096", "--num_nodes", "1",
        "--num_gpus_per_node", str(gpus), "--memory_constraint", "170", "--mixed_precision", "bf16", "--sequence_parallel",
        "--default_dp_type", "zero2", "--pipeline_type", "pipedream_flush", "--grad_dtype", "bf16",
        "--check_cost_model", "%d,4,1" % (8 * gpus)])
    capsys.readouterr()
    row = next(r for r in table if r["strategy"] == "1-1-%d" % gpus)
    predicted_gib = row["stage_memory_mb"][0] / 1024
    assert abs(predicted_gib - measured_gib) / measured_gib < 0.02


@pytest.mark.parametrize("family,size,layer_mb", [("llama", "llama-7b", [772.0]), ("gpt", "gpt-1.5b", [117.2]), ("bert", "bert-large", [48.0]),
                                                   ("t5", "t5-large", [48.0, 64.0])])
def test_shipped_memory_profiles_carry_the_true_parameter_size(family, size, layer_mb):
    """parameter_size is MB of fp32 parameters of one layer: 12 h^2 for GPT / BERT blocks, 4 h^2 + 3 h f for Llama,
    8 h^2 + ... for T5 encoder / decoder blocks. The profile derives it from measured model states."""
    import json

    here = os.path.join(MODELS, family + "_programs", "configs")
    path = glob.glob(os.path.join(here, "memory_profiling_bf16_*.json"))[0]
    cfg = json.load(open(path))
    sizes = [list(cfg[k].values())[0]["parameter_size"] for k in sorted(cfg) if k.startswith("layertype_")]
    assert len(sizes) == len(layer_mb)
    for got, want in zip(sizes, layer_mb):
        assert abs(got - want) / want < 0.01


@pytest.mark.parametrize("family,size,sp", [("gpt", "gpt-1.5b", True), ("bert", "bert-large", True), ("t5", "t5-large", True),
                                            ("vit", "vit-huge", False), ("swin", "swin-large-patch4-window12-384", False)])
def test_search_runs_from_the_shipped_profiles_of_every_family(family, size, sp, tmp_path, capsys):
    """A user of any family can search without profiling first: the shipped time / memory profiles (measured on two GPUs,
    tensor-parallel degrees 1 and 2) and hardware tables are enough for an 8-GPU search."""
    import json

    from hetu_galvatron_b200.models.runner import search

    argv = ["--model_size", size, "--num_nodes", "1", "--num_gpus_per_node", "8", "--memory_constraint", "40",
            "--mixed_precision", "bf16", "--pipeline_type", "pipedream_flush", "--default_dp_type", "zero2", "--min_bsz", "64",
            "--max_bsz", "64", "--bsz_scale", "1", "--search_space", "full", "--max_tp_deg", "2",
            "--output_config_path", str(tmp_path), "--log_dir", str(tmp_path / "logs")]
    if sp:
        argv.append("--sequence_parallel")
    throughput = search(family, argv=argv)
    capsys.readouterr()
    assert throughput and throughput > 0
    plans = glob.glob(os.path.join(str(tmp_path), "galvatron_config_*.json"))
    assert len(plans) == 1
    plan = json.load(open(plans[0]))
    assert plan["global_bsz"] == 64 and max(int(t) for t in plan["tp_sizes_enc"].split(",")) <= 2
