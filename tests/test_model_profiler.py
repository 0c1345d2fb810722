"""Model profiler: enumeration of measurement points and the derivation of the search engine's keys from raw
measurements (synthetic raw data built from a known linear model, so every derived value is known in closed form)."""
import argparse
import json
import os

import pytest

from hetu_galvatron_b200.profiler.arguments import galvatron_profile_args
from hetu_galvatron_b200.profiler.model_profiler import ModelProfiler, raw_key, stage_cost


def make_args(**kw):
    p = galvatron_profile_args(argparse.ArgumentParser())
    p.add_argument("--seq_length", type=int, default=512)
    p.add_argument("--num_hidden_layers", type=int, default=4)
    p.add_argument("--model_size", type=str, default="llama-7b")
    a = p.parse_args([])
    for k, v in kw.items():
        setattr(a, k, v)
    return a


def test_raw_key_and_stage_cost():
    assert raw_key([1, 2], 8, "seq128", 0, "ms") == "layernum[1,2]_bsz8_seq128_rank0_ms"
    assert raw_key(3, 4, 256) == "layernum3_bsz4_seq256"
    assert stage_cost(2, 2, [1.0, 10.0], 0) == 2.0 and stage_cost(2, 2, [1.0, 10.0], 1) == 20.0


def test_computation_points_and_processing(tmp_path):
    a = make_args(profile_type="computation", profile_mode="batch", profile_min_batch_size=2, profile_max_batch_size=4,
                  profile_batch_size_step=2, layernum_min=2, layernum_max=4, profile_seq_length_list="512")
    prof = ModelProfiler(a)
    prof.set_profiler_launcher(str(tmp_path), ["num_hidden_layers"], "toy")
    pts = prof.computation_points()
    assert [(p["num_hidden_layers"], p["global_train_batch_size"]) for p in pts] == [(2, 2), (2, 4), (4, 2), (4, 4)]
    assert all(p["seq_length"] == 512 and p["pp_deg"] == 1 for p in pts)
    argv = prof.point_argv(pts[0])
    assert "--profile_forward" in argv and argv[argv.index("--profile_forward") + 1] == "1"
    assert "--profile_type" not in argv and "--model_size" in argv
    # raw: time = bsz * (layers * 3.0 + 5.0) ms
    raw = {raw_key([L], b, "seq512"): b * (L * 3.0 + 5.0) for L in (2, 4) for b in (2, 4)}
    json.dump(raw, open(prof.time_profiling_path(), "w"))
    prof.process_profiled_data()
    out = json.load(open(prof.time_profiling_path()))
    assert "bct_fct_coe" not in out            # no whole-iteration measurements in this file
    for b in (2, 4):
        assert out["layertype_0_bsz%d_seq512" % b] == pytest.approx(3.0)
        assert out["layertype_other_bsz%d_seq512" % b] == pytest.approx(5.0)


def test_memory_points_enumeration(tmp_path, monkeypatch):
    monkeypatch.setenv("NUM_NODES", "1")
    monkeypatch.setenv("NUM_GPUS_PER_NODE", "4")
    a = make_args(profile_type="memory", profile_mode="static", profile_batch_size=8, layernum_min=1, layernum_max=2,
                  profile_seq_length_list="512", max_tp_deg=4)
    prof = ModelProfiler(a)
    prof.set_profiler_launcher(str(tmp_path), ["num_hidden_layers"], "toy")
    pts = prof.memory_points()
    combos = {(p["pp_deg"], p["global_tp_deg"], p["global_checkpoint"], p["vocab_tp"], p["num_hidden_layers"]) for p in pts}
    assert (1, 1, 0, 1, 1) in combos and (1, 1, 0, 1, 2) in combos and (1, 1, 1, 1, 2) in combos
    assert (1, 2, 0, 1, 1) in combos and (1, 2, 0, 2, 2) in combos and (1, 4, 0, 4, 1) in combos
    assert (1, 2, 1, 1, 1) not in combos                       # checkpointing only measured at tp 1
    assert (2, 2, 0, 2, 2) in combos and (4, 1, 0, 1, 4) in combos and (4, 2, 0, 1, 4) not in combos
    cmd = prof.launch_command(pts[0])
    assert "torch.distributed.run" in cmd and cmd[cmd.index("--master-addr") + 1] == "127.0.0.1"


@pytest.mark.parametrize("layout", ["fsdp", "engine"])
def test_memory_processing_recovers_the_generating_model(tmp_path, monkeypatch, layout):
    """Raw numbers generated from: per-layer parameter size P/tp (16 bytes per parameter of model states = 4 P, of which
    a rank keeps ``share(dp)``), activation A/tp per sample, other states E and other activation H per sample. Under the
    'fsdp' layout a ZeRO-3 rank keeps 1/dp of the states; under the 'engine' layout what this package's engine keeps
    once an iteration has settled."""
    from hetu_galvatron_b200.search.cost_model import engine_state_ratio

    monkeypatch.setenv("NUM_NODES", "1")
    monkeypatch.setenv("NUM_GPUS_PER_NODE", "4")
    world, bsz, P, A, Ac, E, H = 4, 8, 100.0, 40.0, 6.0, 300.0, 20.0
    a = make_args(profile_type="memory", profile_mode="static", profile_batch_size=bsz, layernum_min=1, layernum_max=2,
                  profile_seq_length_list="512", max_tp_deg=4, profile_dp_type="zero3", memory_layout=layout)
    prof = ModelProfiler(a)
    prof.set_profiler_launcher(str(tmp_path), ["num_hidden_layers"], "toy")
    raw = {}

    def share(d):
        return 1.0 / d if layout == "fsdp" else engine_state_ratio("zero3", d, True, 4, settled=True)

    def fill(pp, tp, ckpt, vtp, layers):
        dp = world // pp // tp
        key = "%d_%d_%d" % (pp, tp, dp) + ("_c" if ckpt else "") + ("_vtp" if vtp and tp > 1 else "")
        entry = raw.setdefault(key, {})
        per_stage = layers // pp
        vt = tp if vtp else 1
        for rank in (0, world - 1):
            ms = per_stage * 4 * P / tp * share(dp) + E / vt * share(world // pp // vt)
            act = per_stage * (Ac if ckpt else A) / tp * (bsz / dp) + H / vt * (bsz / dp)
            entry[raw_key([layers], bsz, "seq512", rank, "ms")] = ms
            entry[raw_key([layers], bsz, "seq512", rank, "act")] = act
            entry[raw_key([layers], bsz, "seq512", rank, "act_peak")] = act

    for p in prof.memory_points():
        fill(p["pp_deg"], p["global_tp_deg"], p["global_checkpoint"], p["vocab_tp"] == p["global_tp_deg"], p["num_hidden_layers"])
    json.dump(raw, open(prof.memory_profiling_path(), "w"))
    prof.process_profiled_data()
    out = json.load(open(prof.memory_profiling_path()))
    layer = out["layertype_0"]["512"]
    assert layer["parameter_size"] == pytest.approx(P)
    acts = layer["tp_activation_per_bsz_dict"]
    assert acts["1"] == pytest.approx(A) and acts["2"] == pytest.approx(A / 2) and acts["4"] == pytest.approx(A / 4)
    assert acts["checkpoint"] == pytest.approx(Ac)
    off = out["other_memory_pp_off"]["512"]
    assert off["model_states"]["1"] == pytest.approx(E) and off["activation"]["1"] == pytest.approx(H)
    assert off["model_states"]["2"] == pytest.approx(E / 2) and off["activation"]["4"] == pytest.approx(H / 4)
    first = out["other_memory_pp_on_first"]["512"]
    assert first["model_states"]["1"] == pytest.approx(E) and first["activation"]["1"] == pytest.approx(H)
    assert "other_memory_pp_on_last" in out


def test_launch_uses_injected_runner(tmp_path):
    a = make_args(profile_type="computation", profile_mode="static", profile_batch_size=4, layernum_min=1, layernum_max=2,
                  profile_seq_length_list="128")
    prof = ModelProfiler(a)
    prof.set_profiler_launcher(str(tmp_path), ["num_hidden_layers"], "toy")
    seen = []
    prof.runner = seen.append
    prof.launch_profiling_scripts()
    assert [p["num_hidden_layers"] for p in seen] == [1, 2, 1, 2]
    assert [p.get("save_profiled_iteration", 0) for p in seen] == [0, 0, 1, 1]


def test_backward_forward_ratio_from_iteration_times(tmp_path):
    a = make_args(profile_type="computation", profile_mode="static", profile_batch_size=2, layernum_min=2, layernum_max=4,
                  profile_seq_length_list="512")
    prof = ModelProfiler(a)
    prof.set_profiler_launcher(str(tmp_path), ["num_hidden_layers"], "toy")
    # forward 3 ms / layer / sample, whole iteration 3 + 6.6 ms / layer / sample (+ constant parts)
    raw = {raw_key([2], 2, "seq512"): 2 * (2 * 3.0 + 5.0), raw_key([4], 2, "seq512"): 2 * (4 * 3.0 + 5.0),
           raw_key([2], 2, "seq512") + "_iter": 2 * (2 * 9.6 + 20.0), raw_key([4], 2, "seq512") + "_iter": 2 * (4 * 9.6 + 20.0)}
    json.dump(raw, open(prof.time_profiling_path(), "w"))
    prof.process_profiled_data()
    out = json.load(open(prof.time_profiling_path()))
    assert out["bct_fct_coe"] == pytest.approx(2.2)
    assert "optimizer_ms_layertype_0" not in out
    # with the optimizer step timed on its own (1.5 ms per layer and step + 4 ms for the rest of the model) it leaves the ratio
    raw[raw_key([2], 2, "seq512") + "_opt"] = 2 * 1.5 + 4.0
    raw[raw_key([4], 2, "seq512") + "_opt"] = 4 * 1.5 + 4.0
    json.dump(raw, open(prof.time_profiling_path(), "w"))
    prof.process_profiled_data()
    out = json.load(open(prof.time_profiling_path()))
    assert out["optimizer_ms_layertype_0"] == pytest.approx(1.5)
    assert out["bct_fct_coe"] == pytest.approx((2 * 2 * 9.6 - 2 * 1.5 - 2 * 2 * 3.0) / (2 * 2 * 3.0))
    assert [k for k in out if k.startswith("layertype_0_")] == ["layertype_0_bsz2_seq512"]      # what the search reads as forward time


def test_two_layer_types_carry_their_own_sequence_lengths(tmp_path):
    """T5: one profile length per layer type, handed to the measured job as --encoder_seq_length / --decoder_seq_length
    (reference: models/T5/arguments.py:36-37 names these two as the sequence length flags of the family)."""
    a = make_args(profile_type="computation", profile_mode="static", profile_batch_size=4, layernum_min=1, layernum_max=2,
                  profile_seq_length_list="512,128")
    prof = ModelProfiler(a)
    prof.set_profiler_launcher(str(tmp_path), ["num_encoder_layers", "num_decoder_layers"], "toy",
                               seqlen_arg_names=["encoder_seq_length", "decoder_seq_length"])
    pts = prof.computation_points()
    assert {(p["num_encoder_layers"], p["num_decoder_layers"]) for p in pts} == {(1, 1), (2, 1), (1, 2)}
    assert all(p["encoder_seq_length"] == 512 and p["decoder_seq_length"] == 128 and "seq_length" not in p for p in pts)
    argv = prof.point_argv(pts[0])
    assert argv[argv.index("--encoder_seq_length") + 1] == "512" and argv[argv.index("--decoder_seq_length") + 1] == "128"
    assert argv[argv.index("--set_seqlen_manually") + 1] == "1"
