"""Unit checks of the pieces around the search: string / JSON codecs, bandwidth readers, latency-table fit, pipeline
division, batch-size sweep and profile ingestion (the reference covers these in tests/core/test_utils.py,
tests/search_engine/test_bsz_utils.py, test_pp_utils.py, test_get_configs.py and test_initialize.py). CPU only."""
import json
import os

import numpy as np
import pytest

from hetu_galvatron_b200.search.cost_model_args import ModelArgs, ParallelArgs, ProfileModelArgs, TrainArgs
from hetu_galvatron_b200.search.search_engine import (check_optimal_chunks, get_cost_all_stages, get_layer_costs,
                                                      get_pp_stage_for_bsz, optimal_chunk_func_default, pp_division_even,
                                                      pp_division_memory_balanced)
from hetu_galvatron_b200.utils import config_utils as cu
from hetu_galvatron_b200.utils import strategy_utils as su
from search_utils import make_engine


# ---------------------------------------------------------------------------------------------- codecs
def test_array_and_json_codecs(tmp_path):
    assert cu.str2array("1,2,4,8") == [1, 2, 4, 8] and cu.str2array("") == []
    assert cu.array2str([2, 2.0, np.int64(4)]) == "2,2,4"
    path = str(tmp_path / "a" / "b" / "cfg.json")
    cu.write_json_config({"x": 1, "y": [1, 2]}, path)                          # creates the folders
    assert cu.read_json_config(path) == {"x": 1, "y": [1, 2]}
    assert cu.num2str(8, "bsz") == "bsz8" and cu.num2str([2048], "seq") == "seq2048"
    assert cu.num2str([4, 8], "layernum") == "layernum[4,8]"
    assert cu.dict_join_dirname({"a": "x.json"}, "/d") == {"a": os.path.join("/d", "x.json")}


@pytest.mark.parametrize("strategy,text", [
    ([1, 1, 8, {"fsdp": 0}], "1-1-8"), ([1, 1, 8, {"fsdp": 1}], "1-1-8f"), ([2, 2, 2, {"tp": 1, "fsdp": 0}], "2-2*-2"),
    ([2, 2, 2, {"tp": 0, "fsdp": 1}], "2-2-2f*"), ([1, 4, 2, {"tp": 1, "fsdp": 1, "cpt": 1}], "1-4*-2f-c"),
    ([1, 4, 2, {"tp": 1, "fsdp": 0, "sp": 1}], "1-4*-2-sp"), ([1, 8, 1, {"cpt": 1, "sp": 1}], "1-8-1-c-sp"),
])
def test_strategy_string_round_trip(strategy, text):
    assert su.form_strategy(strategy) == text
    back = su.strategy_str2list(text)
    assert back[:3] == strategy[:3]
    assert su.form_strategy(back) == text
    assert su.strategy_flags(back) == su.strategy_flags(strategy)


def test_strategy_list_printing(capsys):
    a, b = [1, 2, 4, {"tp": 1, "fsdp": 0}], [1, 1, 8, {"fsdp": 1}]
    assert su.strategies_to_string([a, b]) == "1-2*-4, 1-1-8f"
    assert su.strategies_to_string([[a], [b, b]]) == "1-2*-4 || 1-1-8f, 1-1-8f"
    assert su.strategies_to_string(None) == "None"
    su.print_strategies([a, b])
    assert capsys.readouterr().out.strip() == "1-2*-4, 1-1-8f"


def test_plan_json_round_trip_and_optional_keys():
    layers = [[2, 2, 2, {"tp": 1, "fsdp": 0}], [2, 4, 1, {"fsdp": 0, "sp": 1}], [2, 1, 4, {"fsdp": 1, "cpt": 1}]]
    cfg = cu.strategy2config(layers)
    assert cfg == {"pp_deg": 2, "tp_sizes_enc": "2,4,1", "tp_consecutive_flags": "1,1,1", "dp_types_enc": "0,0,1", "use_sp": "0,1,0"}
    pp, tp, cp, consec, dpt, sp, vtp, vsp, vcp = cu.config2strategy(cfg)
    assert (pp, tp, cp, consec, dpt, sp, vtp, vsp, vcp) == (2, [2, 4, 1], [1, 1, 1], [1, 1, 1], [0, 0, 1], [0, 1, 0], 1, 0, 1)
    cfg.update(cp_sizes_enc="1,2,1", vtp=4, vsp=1, vcp=2)
    assert cu.config2strategy(cfg)[2] == [1, 2, 1] and cu.config2strategy(cfg)[6:] == (4, 1, 2)
    assert cu.strategy2config([]) == {}


def test_bandwidth_readers():
    env = {"allreduce_size_8_consec_1": 160.0, "allreduce_size_4_consec_0": 150.0, "allreduce_size_4_consec_1": 155.0,
           "allreduce_size_2_consec_0": 140.0, "allreduce_size_2_consec_1": 145.0}
    bw, coe = cu.read_allreduce_bandwidth_config(env, 8)
    assert set(bw) == {"8", "4_0", "4_1", "2_0", "2_1", "1"}
    assert coe["8"] == pytest.approx(1 / 160) and coe["2_0"] == pytest.approx(1 / 140) and coe["1"] == 0 and bw["1"] == np.inf
    bw4, _ = cu.read_allreduce_bandwidth_config(env, 4)
    assert set(bw4) == {"4", "2_0", "2_1", "1"} or "4" not in bw4      # a 4-GPU file names its top group 4_consec_1
    p2p, pcoe = cu.read_p2p_bandwidth_config({"pp_size_2": 200.0, "pp_size_4": 100.0, "note": 1})
    assert p2p == {2: 200.0, 4: 100.0} and pcoe[4] == pytest.approx(0.01)


def test_latency_table_fit():
    table = {}
    for world in (2, 4):
        for mb in (1, 2, 4, 8, 16, 32, 64, 128):
            table["allreduce_size_%d_%dMB_time" % (world, mb)] = 2 * (0.01 * world * mb + 0.05)
            table["all2all_size_%d_%dMB_time" % (world, mb)] = 0.003 * mb + 0.02
    ar = cu.remap_config(table, "allreduce")
    assert sorted(ar) == [2, 4] and ar[2][4 * 2 ** 20] == pytest.approx(0.01 * 2 * 4 + 0.05)   # halved: one all-gather
    assert ar[4]["popt"] == pytest.approx([0.04, 0.05], rel=1e-5)
    a2a = cu.remap_config(table, "all2all")
    assert a2a[2]["popt"] == pytest.approx([0.003, 0.02], rel=1e-5) and a2a[4][128 * 2 ** 20] == pytest.approx(0.003 * 128 + 0.02)
    with pytest.raises(AssertionError):
        cu.remap_config({"allreduce_size_2_1MB_time": 1.0}, "allreduce")


# ---------------------------------------------------------------------------------------------- chunks / division
def test_default_chunk_rule():
    assert optimal_chunk_func_default(32, [1, 1, 8, {}], 4, 1) == 8
    assert optimal_chunk_func_default(32, [1, 4, 2, {}], 4, 2) == 4          # tp above min_tp shrinks the local batch
    assert optimal_chunk_func_default(2, [1, 8, 1, {}], 4, 1) == 1            # never zero
    chunks = check_optimal_chunks(8, [[1, 1, 8, {}], [2, 1, 4, {}], [4, 2, 1, {}]], optimal_chunk_func_default, 64,
                                  {1: 4, 2: 2, 4: 1}, 1)
    assert chunks == {1: 2, 2: 8, 4: 32}


def test_even_division_and_stage_sums():
    assert pp_division_even([28], 4) == [7, 7, 7, 7] and pp_division_even([30], 4) == [7, 7, 7, 9]
    assert pp_division_even([12, 12], 2) == [12, 12] and pp_division_even([5], 1) == [5]
    assert get_layer_costs([2, 3], [1.5, 4.0]) == [1.5, 1.5, 4.0, 4.0, 4.0]
    assert get_cost_all_stages([1, 2, 3, 4], [2, 2]) == [3, 7]
    assert get_cost_all_stages([10, 1, 2, 3, 4], [2, 2]) == [13, 7]            # + embedding on the first stage
    assert get_cost_all_stages([10, 1, 2, 3, 4, 20], [2, 2]) == [13, 27]       # + head on the last


def _division_args(params):
    n = len(params)
    other_off = {"model_states": {1: 2000.0}, "activation": {1: 50.0}}
    other_on = {"first_stage": {"model_states": {1: 1200.0}, "activation": {1: 20.0}},
                "last_stage": {"model_states": {1: 800.0}, "activation": {1: 30.0}}}
    return ([ModelArgs(parameter_size=p) for p in params], [TrainArgs(mixed_precision=True, pytorch_context_mem=512)] * n,
            [ParallelArgs(chunks=4) for _ in range(n)],
            [ProfileModelArgs(tp_activation_per_bsz_dict={1: 30.0 * (i + 1), "checkpoint": 4.0}, other_memory_pp_off=other_off,
                              other_memory_pp_on=other_on) for i in range(n)])


@pytest.mark.parametrize("layers,params,pp", [([24], [48.0], 4), ([12, 12], [40.0, 120.0], 2), ([6, 18], [200.0, 30.0], 4),
                                               ([2, 2, 18, 2], [20.0, 40.0, 80.0, 160.0], 4)])
def test_memory_balanced_division(layers, params, pp):
    m, t, p, pm = _division_args(params)
    strategies = [[pp, 1, 8 // pp, {"fsdp": 0}], [1, 1, 8, {"fsdp": 0}]]
    divide, mem = pp_division_memory_balanced(m, t, p, pm, layers, pp, 32, 2, strategies)
    assert sum(divide) == sum(layers) and len(divide) == pp and all(d >= 1 for d in divide)
    assert len(mem) == pp
    # no stage far above the mean (the last one takes what is left)
    assert max(mem[:-1]) <= 1.3 * np.mean(mem) + 1e-6
    if len(layers) == 1:                       # embedding and head weigh on the end stages, which get fewer layers
        assert divide[0] <= divide[1] and divide[-1] <= divide[-2]
    one, none = pp_division_memory_balanced(m, t, p, pm, layers, 1, 32, 2, strategies)
    assert one == [sum(layers)] and none is None
    assert pp_division_memory_balanced(m, t, p, pm, layers, 8, 32, 2, strategies) == (None, None)


def test_heavier_layers_get_fewer_per_stage():
    m, t, p, pm = _division_args([30.0, 300.0])
    divide, _ = pp_division_memory_balanced(m, t, p, pm, [12, 12], 2, 32, 2, [[2, 1, 4, {"fsdp": 0}]])
    assert divide[0] > divide[1]


def test_stage_table_for_every_pp_degree():
    m, t, p, pm = _division_args([48.0])
    strategies = [[1, 1, 8, {}], [2, 1, 4, {}], [4, 1, 2, {}]]
    table = get_pp_stage_for_bsz(strategies, m, t, p, pm, [24], 32, {1: 2, 2: 2, 4: 2})
    assert table == {1: [24], 2: [12, 12], 4: [6, 6, 6, 6]}
    table = get_pp_stage_for_bsz(strategies, m, t, p, pm, [24], 32, {1: 2, 2: 2, 4: 2}, single_layer_even=False)
    assert sorted(table) == [1, 2, 4] and all(sum(v) == 24 for v in table.values())


# ---------------------------------------------------------------------------------------------- engine set-up
def test_batch_size_sweep(tmp_path):
    eng, _ = make_engine(str(tmp_path), settle_bsz=48)
    eng.set_searching_bsz()
    assert eng.BSZs == [48] and eng.min_bsz == eng.max_bsz == 48
    eng.args.settle_bsz, eng.args.min_bsz, eng.args.max_bsz, eng.args.bsz_scale = -1, 20, 64, 16
    eng.set_searching_bsz()
    assert eng.BSZs == [16, 32, 48, 64] and eng.max_bsz == 64
    eng.args.max_bsz = 70
    eng.set_searching_bsz()
    assert eng.BSZs[-1] == 64 and eng.BSZs[0] == 16
    eng.args.min_bsz, eng.args.bsz_scale = 4, 8                                 # below one step: start at the step
    eng.set_searching_bsz()
    assert eng.BSZs[0] == 8


def test_recommended_start_lies_between_the_pure_strategies(tmp_path):
    eng, _ = make_engine(str(tmp_path), memory_constraint=36)
    limits = [eng.estimate_strategy_max_bsz([s], 8) for s in ([1, 1, 8, {"fsdp": 0}], [1, 1, 8, {"fsdp": 1}], [1, 8, 1, {"fsdp": 0}])]
    rec = eng.recommend_min_bsz(8)
    assert rec % 8 == 0 and rec >= 8
    assert min(limits) <= max(rec, min(limits)) <= max(max(limits), 8)
    eng.args.search_space = "sdp"
    assert eng.recommend_min_bsz(8) == -1


def test_profile_ingestion_static(tmp_path):
    eng, _ = make_engine(str(tmp_path))
    assert eng.layernum_list == [28] and eng.num_layertype == 1 and eng.seqlen_list == [4096]
    assert len(eng.model_args_list) == len(eng.train_args_list) == len(eng.parallel_args_list) == 1
    assert len(eng.profile_model_args_list) == len(eng.profile_hardware_args_list) == 1
    pm = eng.profile_model_args_list[0]
    acts = pm.tp_activation_per_bsz_dict
    assert acts[1] > acts[2] > acts[4] > acts[8] > 0 and acts["checkpoint"] < acts[8]
    assert set(pm.other_memory_pp_on) == {"first_stage", "last_stage"}
    assert eng.model_args_list[0].parameter_size > 0 and eng.model_args_list[0].hidden_size == 3584
    hw = eng.profile_hardware_args_list[0]
    assert set(hw.comm_coe_dict) >= {"8", "4_0", "4_1", "2_0", "2_1", "1"} and hw.comm_coe_dict["1"] == 0
    assert set(hw.p2p_comm_coe_dict) == {2, 4, 8}
    assert hw.dp_overlap_coe >= 1.0 and hw.bct_overlap_coe >= 1.0
    assert sorted(hw.allreduce_dict) == [2, 4, 8] and "popt" in hw.allreduce_dict[2]
    assert eng.memory_constraint == 24 * 1024


def test_profile_ingestion_sequence_mode(tmp_path):
    eng, _ = make_engine(str(tmp_path), time_mode="sequence", memory_mode="sequence", sp=True, seqlen_list=[8192])
    pm = eng.profile_model_args_list[0]
    assert pm.tp_activation_per_bsz_dict[1] > pm.tp_activation_per_bsz_dict[8] > 0
    fct = pm.forward_computation_time
    assert np.all(np.asarray(fct) > 0) if np.ndim(fct) == 0 else float(np.asarray(fct).ravel()[0]) > 0


def test_search_emits_a_loadable_plan(tmp_path):
    from hetu_galvatron_b200.core.plan import HybridPlan

    eng, out = make_engine(str(tmp_path), settle_bsz=32, settle_chunk=4, memory_constraint=36)
    throughput = eng.parallelism_optimization()
    assert throughput > 0
    files = [f for f in os.listdir(out) if f.startswith("galvatron_config_")]
    assert len(files) == 1
    cfg = json.load(open(os.path.join(out, files[0])))
    assert cfg["global_bsz"] == 32 and cfg["chunks"] >= 1 and len(cu.str2array(cfg["tp_sizes_enc"])) == 28
    assert sum(cu.str2array(cfg["pp_division"])) == 28 and cfg["pipeline_type"] in ("gpipe", "pipedream_flush")
    plan = HybridPlan.from_json(os.path.join(out, files[0]), 28)
    assert plan.pp_deg == cfg["pp_deg"] and len(plan.tp_sizes_enc) == 28 and plan.chunks == cfg["chunks"]


def test_explain_plan_prices_a_searched_plan_like_the_search_did(tmp_path):
    eng, out = make_engine(str(tmp_path), settle_bsz=32, settle_chunk=4, memory_constraint=36)
    throughput = eng.parallelism_optimization()
    plan = json.load(open(eng.output_path))
    report = eng.explain_plan(plan)
    assert len(report["stage_memory_mb"]) == plan["pp_deg"] == len(report["stage_time_s"])
    assert len(report["strategies"]) == 28
    # layers + embedding / head under the limit the search was given (it reserves 20 % for the allocator)
    assert max(report["stage_memory_mb"]) <= 36 * 1024
    # the layer part of the step the search minimised (its total adds embedding / head time)
    assert 0.5 * 32 / throughput < report["step_time_s"] <= 32 / throughput * 1.001
    assert report["throughput_samples_per_s"] == pytest.approx(32 / report["step_time_s"])
    # a hand-written uniform plan: more tensor parallelism means less memory per rank
    def uniform(tp):
        n = 28
        return {"pp_deg": 1, "tp_sizes_enc": ",".join([str(tp)] * n), "tp_consecutive_flags": ",".join(["1"] * n),
                "dp_types_enc": ",".join(["0"] * n), "use_sp": ",".join(["0"] * n), "checkpoint": ",".join(["0"] * n),
                "global_bsz": 32, "chunks": 4, "pp_division": str(n), "vtp": tp, "vsp": 0, "embed_sdp": 0}
    m2, m8 = eng.explain_plan(uniform(2)), eng.explain_plan(uniform(8))
    assert m8["stage_memory_mb"][0] < m2["stage_memory_mb"][0]
    assert m2["strategies"][0] == "1-2*-4" and m8["strategies"][0] == "1-8-1"


def test_capped_table_gives_the_same_answers_as_the_full_table():
    """The solver only builds the table up to the sum of the layers' largest feasible memory costs (above it the budget
    binds nowhere). Costs, plans and remaining memory equal those of the full table, for both cores, with ties, with
    strategies that never fit and with vocab keys that start above, inside and below the table."""
    import numpy as np

    from hetu_galvatron_b200.search.dynamic_programming import DPAlg

    rng = np.random.RandomState(1)
    capped_some = False
    for trial in range(120):
        L, S, V = rng.randint(1, 7), rng.randint(1, 6), rng.randint(5, 120)
        v = rng.randint(0, 30, (L, S))
        if rng.rand() < 0.3:
            v[rng.randint(L), rng.randint(S)] = V + rng.randint(0, 50)
        inter, intra = np.round(rng.rand(L, S, S) * 4) / 4, np.round(rng.rand(L, S) * 8) / 4
        other_mem, other_time = {1: int(rng.randint(0, V + 10)), 2: int(rng.randint(0, 40))}, {1: 0.5, 2: 1.5}
        outs = []
        for cpp in (True, False):
            for capped in (True, False):
                dp = DPAlg(V, dict(other_mem), dict(other_time), L, S, None, True, use_cpp_core=cpp)
                dp.set_v_and_cost(v, intra, inter)
                outs.append(dp._fit_capped() if capped else dp._fit_table())
        capped_some |= int(np.where(v < V + 1, v, 0).max(axis=1).sum()) + 1 < V + 1
        for total, res, remain in outs:
            for k in other_mem:
                assert total[k] == outs[1][0][k] and list(res[k]) == list(outs[1][1][k]) and remain[k] == outs[1][2][k], (trial, k)
    assert capped_some
