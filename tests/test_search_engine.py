"""Search engine: strategy space, golden end-to-end searches on canned A100-era profiles, C++ core vs NumPy DP.

The golden throughputs / plans are the values the reference pins for the same inputs
(tests/search_engine/test_parallelsim_optimization.py:35,85; test_generate_strategies.py:46)."""
import glob
import json
import os

import numpy as np
import pytest

from hetu_galvatron_b200.search import DPAlg, GalvatronSearchEngine
from hetu_galvatron_b200.utils import print_strategies
from hetu_galvatron_b200.utils.strategy_utils import strategies_to_string
from search_utils import LLAMA_SEARCH_LAYERS, make_engine, search_args

FULL_TP_SP = ("1-1-8, 1-1-8f, 1-2-4*, 1-2-4*-sp, 1-2-4f*, 1-2-4f*-sp, 1-2*-4, 1-2*-4-sp, 1-2*-4f, 1-2*-4f-sp, 1-4-2*, 1-4-2*-sp, "
              "1-4-2f*, 1-4-2f*-sp, 1-4*-2, 1-4*-2-sp, 1-4*-2f, 1-4*-2f-sp, 1-8-1, 1-8-1-sp, 2-1-4, 2-1-4f, 2-2-2*, 2-2-2*-sp, "
              "2-2-2f*, 2-2-2f*-sp, 2-2*-2, 2-2*-2-sp, 2-2*-2f, 2-2*-2f-sp, 2-4-1, 2-4-1-sp, 4-1-2, 4-1-2f, 4-2-1, 4-2-1-sp, 8-1-1")


@pytest.mark.parametrize("space", ["dp+tp", "dp+pp", "3d", "dp", "tp", "pp", "sdp", "full"])
@pytest.mark.parametrize("sp_space", ["tp", "sp", "tp+sp"])
def test_generate_strategies(space, sp_space, tmp_path):
    eng = GalvatronSearchEngine(search_args(search_space=space, sp_space=sp_space))
    eng.set_search_engine_info(str(tmp_path), LLAMA_SEARCH_LAYERS, "m")
    eng.generate_strategies()
    assert len(eng.strategies) > 0
    if space == "full" and sp_space == "tp+sp":
        assert len(eng.strategies) == 74
        plain = FULL_TP_SP.split(", ")
        with_ckpt = [s + "-c" if not s.endswith("-sp") else s[:-3] + "-c-sp" for s in plain]
        assert strategies_to_string(eng.strategies) == ", ".join(plain + with_ckpt)


GOLD = dict(settle_bsz=64, sp_space="tp+sp", memory_constraint=36, default_dp_type="zero2", pipeline_type="pipedream_flush",
            async_grad_reduce=False, sequence_parallel=True)


def test_golden_fine_grained_search(tmp_path):
    eng, out = make_engine(str(tmp_path), "sequence", "sequence", True, [8192], settle_chunk=32, fine_grained_mode=1, **GOLD)
    thr = eng.parallelism_optimization()
    assert abs(thr - 2.8074257503114315) < 1e-6
    files = glob.glob(os.path.join(out, "*.json"))
    assert len(files) == 1 and os.path.basename(files[0]).startswith("galvatron_config_")
    cfg = json.load(open(files[0]))
    assert cfg["pp_deg"] == 1 and cfg["global_bsz"] == 64 and cfg["chunks"] == 32 and cfg["pp_division"] == "28"
    assert cfg["pipeline_type"] == "pipedream_flush" and cfg["default_dp_type"] == "zero2"
    assert cfg["vtp"] == 8 and cfg["vsp"] == 0 and cfg["embed_sdp"] == 0
    for field, val in {"tp_sizes_enc": "8", "tp_consecutive_flags": "1", "dp_types_enc": "0", "use_sp": "0"}.items():
        assert cfg[field].split(",") == [val] * 28
    assert cfg["checkpoint"] == ",".join(["1"] * 8 + ["0"] * 20)


def test_golden_coarse_search(tmp_path):
    eng, out = make_engine(str(tmp_path), "sequence", "sequence", True, [8192], settle_chunk=8, fine_grained_mode=0, **GOLD)
    thr = eng.parallelism_optimization()
    assert abs(thr - 2.5234175303522344) < 1e-6
    cfg = json.load(open(glob.glob(os.path.join(out, "*.json"))[0]))
    assert cfg["pp_deg"] == 1 and cfg["chunks"] == 8 and cfg["vtp"] == 1 and cfg["vsp"] == 0 and cfg["embed_sdp"] == 1
    for field, val in {"tp_sizes_enc": "1", "tp_consecutive_flags": "1", "dp_types_enc": "1", "use_sp": "0", "checkpoint": "1"}.items():
        assert cfg[field].split(",") == [val] * 28


def test_cpp_core_matches_numpy_dp():
    rng = np.random.default_rng(0)
    L, S, M = 6, 5, 300
    v = rng.integers(0, 60, size=(L, S)).astype(np.int32)       # includes zero-cost cells
    intra = rng.random((L, S))
    inter = rng.random((L, S, S)) * 0.1
    inter[0] = 0
    other_mem = {1: 20, 2: 35, 4: 400}
    other_time = {1: 0.5, 2: 0.25, 4: 0.1}
    outs = []
    for use_cpp in (True, False):
        dp = DPAlg(M, dict(other_mem), dict(other_time), L, S, None, True, use_cpp_core=use_cpp)
        dp.set_v_and_cost(v, intra, inter)
        outs.append(dp.fit())
    (c1, r1, m1), (c2, r2, m2) = outs
    for k in other_mem:
        assert (np.isinf(c1[k]) and np.isinf(c2[k])) or abs(c1[k] - c2[k]) < 1e-12
        assert m1[k] == m2[k]
        if m1[k] >= 0:
            assert list(r1[k]) == list(r2[k])
            assert sum(v[i, r1[k][i]] for i in range(L)) + other_mem[k] + m1[k] == M
    assert m1[4] == -1      # 400 MB of "other" memory does not fit a 300 MB budget


def test_static_search_runs_and_respects_memory(tmp_path):
    eng, out = make_engine(str(tmp_path), "static", "static", False, None, settle_bsz=32, settle_chunk=4, memory_constraint=24,
                           sp_space="tp")
    thr = eng.parallelism_optimization()
    assert thr > 0
    assert max(eng.best_result["mem_cost"]) <= 24 * 1024


def test_context_parallel_as_outer_search_dimension(tmp_path):
    """cp = 1 reproduces the plain search; a long-sequence, memory-bound case prefers cp > 1 and emits a loadable plan."""
    import json
    from hetu_galvatron_b200.core.plan import HybridPlan
    from hetu_galvatron_b200.search.context_parallel import kv_gather_ms_per_sample, search_with_context_parallel
    from search_utils import LLAMA_SEARCH_LAYERS

    assert kv_gather_ms_per_sample(4096, 4096, 1, {"1": 0}) == 0.0
    assert kv_gather_ms_per_sample(4096, 4096, 4, {"4_0": 0.002}) == pytest.approx(3 / 4 * 64.0 * 0.002)
    eng, out = make_engine(str(tmp_path), settle_bsz=16, settle_chunk=2, memory_constraint=36)
    plain = eng.parallelism_optimization()
    res = search_with_context_parallel(eng.args, eng.path, LLAMA_SEARCH_LAYERS, "llama_search", max_cp_deg=1)
    assert res["cp"] == 1 and res["throughput"] == pytest.approx(plain, rel=1e-9)
    # two sequences on eight GPUs with tp <= 2 and no pipeline: without splitting the sequence there is no layout at all
    tight, _ = make_engine(str(tmp_path / "tight"), settle_bsz=2, settle_chunk=1, memory_constraint=24, max_tp_deg=2, disable_pp=1)
    base = search_with_context_parallel(tight.args, tight.path, LLAMA_SEARCH_LAYERS, "llama_search", max_cp_deg=1)
    wide = search_with_context_parallel(tight.args, tight.path, LLAMA_SEARCH_LAYERS, "llama_search", max_cp_deg=4)
    assert sorted(wide["per_cp"]) == [1, 2, 4]
    assert base["throughput"] <= 0 and wide["per_cp"][1] <= 0
    assert wide["throughput"] > 0 and wide["cp"] == 2 and wide["per_cp"][2] > wide["per_cp"][4] > 0
    cfg = json.load(open(wide["path"]))
    assert cfg["vcp"] == wide["cp"] and set(cfg["cp_sizes_enc"].split(",")) == {str(wide["cp"])}
    plan = HybridPlan.from_json(wide["path"], 28)
    plan.validate(8, 28)
    assert plan.cp_sizes_enc == [wide["cp"]] * 28


def _two_layer_type_engine(tmp, memory_gb):
    """Synthetic encoder-decoder profile: 12 + 12 layers, the decoder layers 1.8x slower and 1.5x larger."""
    import json
    import os

    from hetu_galvatron_b200.search import GalvatronSearchEngine
    from search_utils import FIX, search_args

    cfg, hw = os.path.join(tmp, "configs"), os.path.join(tmp, "hw")
    os.makedirs(cfg), os.makedirs(hw)
    name = "encdec"
    json.dump({"layertype_0_bsz1_seq512": 1.0, "layertype_1_bsz1_seq512": 1.8, "layertype_other_bsz1_seq[512,512]": 0.7},
              open(os.path.join(cfg, "computation_profiling_bf16_%s.json" % name), "w"))
    act = lambda k: {"1": 40.0 * k, "2": 22.0 * k, "4": 12.0 * k, "8": 7.0 * k, "checkpoint": 4.0 * k}
    other = {"model_states": {"1": 800.0, "2": 400.0, "4": 200.0, "8": 100.0}, "activation": {"1": 30.0, "2": 16.0, "4": 9.0, "8": 5.0}}
    other_pp = {"model_states": {"1": 400.0, "2": 200.0, "4": 100.0}, "activation": {"1": 15.0, "2": 8.0, "4": 4.5}}
    json.dump({"layertype_0": {"512": {"parameter_size": 48.0, "tp_activation_per_bsz_dict": act(1)}},
               "layertype_1": {"512": {"parameter_size": 64.0, "tp_activation_per_bsz_dict": act(1.5)}},
               "other_memory_pp_off": {"[512,512]": other}, "other_memory_pp_on_first": {"[512,512]": other_pp},
               "other_memory_pp_on_last": {"[512,512]": other_pp}},
              open(os.path.join(cfg, "memory_profiling_bf16_%s.json" % name), "w"))
    src = json.load(open(os.path.join(FIX, "hardware.json")))
    for key, fname in (("allreduce", "allreduce_bandwidth_1nodes_8gpus_per_node.json"), ("p2p", "p2p_bandwidth_1nodes_8gpus_per_node.json"),
                       ("overlap", "overlap_coefficient.json"), ("sp", "sp_time_1nodes_8gpus_per_node.json")):
        json.dump(src[key], open(os.path.join(hw, fname), "w"))
    args = search_args(memory_constraint=memory_gb, settle_bsz=64, settle_chunk=4, time_profiling_path=cfg, memory_profiling_path=cfg,
                       allreduce_bandwidth_config_path=hw, p2p_bandwidth_config_path=hw, overlap_coe_path=hw, sp_time_path=hw,
                       output_config_path=os.path.join(tmp, "out"), log_dir=os.path.join(tmp, "logs"), hidden_size=1024,
                       pipeline_type="pipedream_flush", default_dp_type="zero2")
    eng = GalvatronSearchEngine(args)
    eng.set_search_engine_info(tmp, [{"hidden_size": 1024, "layer_num": 12, "seq_len": 512},
                                     {"hidden_size": 1024, "layer_num": 12, "seq_len": 512}], name)
    eng.initialize_search_engine(show=False)
    return eng


def test_two_layer_types_search_and_memory_pressure(tmp_path):
    """Encoder-decoder models are searched as two layer types (reference T5: pp_division_memory_balanced). With room to
    spare the plan is pure data parallelism; under pressure it must shard, checkpoint or pipeline, at lower throughput."""
    import json

    roomy = _two_layer_type_engine(str(tmp_path / "a"), 8)
    t_roomy = roomy.parallelism_optimization()
    p = json.load(open(roomy.output_path))
    assert p["pp_deg"] == 1 and set(p["tp_sizes_enc"].split(",")) == {"1"} and len(p["tp_sizes_enc"].split(",")) == 24
    tight = _two_layer_type_engine(str(tmp_path / "b"), 3)
    t_tight = tight.parallelism_optimization()
    q = json.load(open(tight.output_path))
    assert 0 < t_tight < t_roomy
    uses = (q["pp_deg"] > 1 or "1" in q["dp_types_enc"].split(",") or "1" in q["checkpoint"].split(",")
            or set(q["tp_sizes_enc"].split(",")) != {"1"})
    assert uses, q
    assert sum(int(x) for x in q["pp_division"].split(",")) == 24
    report = tight.explain_plan(q)
    assert max(report["stage_memory_mb"]) <= 3 * 1024
