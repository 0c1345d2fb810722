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
