"""Driver logic of the runtime and hardware profilers and the flag groups, on CPU with the device calls faked (the
reference checks the same layers in tests/profiler/test_runtime_profile.py:7-230, test_hardware_profile.py:15-156 and
tests/test_arguments.py:7-126). No GPU and no process group are touched."""
import json
import os
from types import SimpleNamespace

import pytest

from hetu_galvatron_b200.core.arguments import get_args, initialize_galvatron
from hetu_galvatron_b200.models.arguments import make_model_args
from hetu_galvatron_b200.profiler import runtime_profiler as rp
from hetu_galvatron_b200.profiler.hardware_profiler import HardwareProfiler
from hetu_galvatron_b200.profiler.utils import memory_strategy_key, save_profiled_memory, save_profiled_time


# ---------------------------------------------------------------------------------------------- flag groups
def test_training_flags_defaults_and_overrides():
    a = initialize_galvatron(make_model_args("llama"), mode="train", argv=[])
    assert a.galvatron_mode == "train" and get_args() is a
    assert a.pp_deg == 2 and a.global_tp_deg == -1 and a.chunks == -1 and a.pipeline_type in ("gpipe", "pipedream_flush")   # the reference's defaults
    assert a.default_dp_type in ("ddp", "zero2", "zero3") and a.mixed_precision in ("fp32", "fp16", "bf16")
    assert a.galvatron_config_path is None and a.make_vocab_size_divisible_by == 128
    a = initialize_galvatron(make_model_args("llama"), mode="train", argv=[
        "--pp_deg", "2", "--global_tp_deg", "4", "--global_train_batch_size", "64", "--chunks", "8", "--sdp", "1",
        "--global_checkpoint", "1", "--pipeline_type", "gpipe", "--default_dp_type", "zero2", "--mixed_precision", "bf16",
        "--sequence-parallel", "--use-ulysses", "--vocab_tp", "2", "--global_cp_deg", "2", "--model_size", "llama-7b",
        "--galvatron_config_path", "plan.json", "--an_unknown_flag", "1"])
    assert (a.pp_deg, a.global_tp_deg, a.global_train_batch_size, a.chunks, a.sdp, a.global_checkpoint) == (2, 4, 64, 8, 1, 1)
    assert a.pipeline_type == "gpipe" and a.default_dp_type == "zero2" and a.sequence_parallel and a.use_ulysses
    assert a.vocab_tp == 2 and a.global_cp_deg == 2 and a.model_size == "llama-7b" and a.galvatron_config_path == "plan.json"


def test_profile_search_and_hardware_flag_groups():
    p = initialize_galvatron(make_model_args("gpt"), mode="profile", argv=["--profile_type", "memory", "--profile_mode", "static",
                                                                            "--profile_batch_size", "4", "--layernum_min", "2",
                                                                            "--layernum_max", "4", "--max_tp_deg", "4"])
    assert (p.profile_type, p.profile_mode, p.profile_batch_size, p.layernum_min, p.layernum_max, p.max_tp_deg) == \
        ("memory", "static", 4, 2, 4, 4)
    s = initialize_galvatron(make_model_args("llama"), mode="search", argv=["--memory_constraint", "160", "--search_space", "dp+tp",
                                                                            "--sp_space", "tp+sp", "--settle_bsz", "64",
                                                                            "--num_gpus_per_node", "8", "--fine_grained_mode", "0",
                                                                            "--check_cost_model", "64,4,1", "--bct_fct_coe", "2.35"])
    assert (s.memory_constraint, s.search_space, s.sp_space, s.settle_bsz, s.fine_grained_mode) == (160, "dp+tp", "tp+sp", 64, 0)
    assert s.check_cost_model == "64,4,1" and s.bct_fct_coe == pytest.approx(2.35) and s.num_nodes == 1
    h = initialize_galvatron(None, mode="profile_hardware", argv=["--num_gpus_per_node", "4", "--max_pp_deg", "4"])
    assert h.num_gpus_per_node == 4 and h.max_pp_deg == 4 and h.galvatron_mode == "profile_hardware"
    with pytest.raises(ValueError):
        initialize_galvatron(None, mode="no_such_mode", argv=[])


# ---------------------------------------------------------------------------------------------- profile files
def test_memory_key_grammar():
    assert memory_strategy_key(1, 1, 8, 0) == "1_1_8"
    assert memory_strategy_key(2, 2, 8, 1) == "2_2_2_c"
    assert memory_strategy_key(1, 4, 8, 0, vocab_tp=4, sequence_parallel=True) == "1_4_2_vtp_sp"
    assert memory_strategy_key(1, 1, 8, 0, vocab_tp=1) == "1_1_8"             # vtp tag only when tp > 1


def test_profile_writers_merge_into_one_file(tmp_path):
    path = str(tmp_path / "configs" / "memory.json")
    save_profiled_memory(path, 1, 2, 8, [2], 8, 0, 100.0, 50.0, 70.0, 0, True, 2, [4096])
    save_profiled_memory(path, 1, 2, 8, [4], 8, 7, 180.0, 90.0, 110.0, 0, True, 2, [4096])
    save_profiled_memory(path, 2, 1, 8, [2, 4], 16, 0, 1.0, 2.0, 3.0, 1, False, 1, [512, 256])
    cfg = json.load(open(path))
    assert set(cfg) == {"1_2_4_vtp_sp", "2_1_4_c"}
    assert cfg["1_2_4_vtp_sp"]["layernum[2]_bsz8_seq4096_rank0_ms"] == 100.0
    assert cfg["1_2_4_vtp_sp"]["layernum[4]_bsz8_seq4096_rank7_act_peak"] == 110.0
    assert cfg["2_1_4_c"]["layernum[2,4]_bsz16_seq[512,256]_rank0_act"] == 2.0
    tpath = str(tmp_path / "configs" / "time.json")
    save_profiled_time(tpath, 12.5, 8, [2], [4096])
    save_profiled_time(tpath, 40.0, 8, [2], [4096], suffix="_iter")
    assert json.load(open(tpath)) == {"layernum[2]_bsz8_seq4096": 12.5, "layernum[2]_bsz8_seq4096_iter": 40.0}


# ---------------------------------------------------------------------------------------------- runtime profiler
def _args(**kw):
    base = dict(profile=1, profile_type="allocated", mixed_precision="bf16", pipeline_type="gpipe", pp_deg=1, global_tp_deg=1,
                global_train_batch_size=8, global_checkpoint=0, sequence_parallel=False, vocab_tp=1, save_profiled_memory=0,
                profile_forward=0, save_profiled_iteration=0, exit_after_profiling=False, lr=1e-4, local_rank=0)
    base.update(kw)
    return SimpleNamespace(**base)


def test_runtime_profiler_memory_bookkeeping(tmp_path, monkeypatch, capsys):
    readings = iter([(0, 100), (0, 160), (230, 110),          # iteration 3: before fwd, after fwd, after bwd (peak 230)
                     (0, 100), (0, 164), (240, 112)])         # iteration 4
    prof = rp.RuntimeProfiler(_args(save_profiled_memory=1), path=str(tmp_path), model_name="m")
    monkeypatch.setattr(prof, "_mem", lambda: next(readings))
    prof.set_profiler_dist(str(tmp_path), [{"hidden_size": 64, "layer_num": 2, "seq_len": 32}], "m", profile_ranks=[0], rank=0)
    for it in (3, 4):
        prof.profile_memory(it, "Before Forward")
        prof.profile_memory(it, "After Forward")
        prof.profile_memory(it, "After Backward")
        prof.post_profile_memory(it)                          # not the last profiled iteration: nothing happens
    prof.profile_memory(9, "Before Forward")                  # past max_profile_iter: ignored
    assert "iter_9_before_forward" not in prof.mem_dict
    with pytest.raises(SystemExit):
        prof.post_profile_memory(5)
    m = prof.mem_dict
    assert m["model_states"] == 112 and m["activation"] == 64 and m["model_states_and_peak_activation"] == 240
    assert m["peak_activation"] == 128 and m["model_states_and_activation"] == 164
    cfg = json.load(open(prof.memory_profiling_path()))
    assert cfg == {"1_1_1": {"layernum[2]_bsz8_seq32_rank0_ms": 112, "layernum[2]_bsz8_seq32_rank0_act": 64,
                             "layernum[2]_bsz8_seq32_rank0_act_peak": 128}}
    assert "Max memory" in capsys.readouterr().out


def test_runtime_profiler_skips_when_disabled(tmp_path):
    prof = rp.RuntimeProfiler(_args(profile=0), path=str(tmp_path), model_name="m")
    prof.profile_memory(1, "Before Forward")
    prof.profile_time_start(1)
    prof.profile_time_end(1, loss=1.0)
    assert prof.mem_dict == {} and prof.time_list == []
    with pytest.raises(AssertionError):
        prof.set_time_profiler(5, 5)


def test_runtime_profiler_time_window_and_outputs(tmp_path, monkeypatch, capsys):
    clock = {"t": 0.0}
    monkeypatch.setattr(rp.time, "perf_counter", lambda: clock["t"])
    monkeypatch.setattr(rp.torch.cuda, "is_available", lambda: False)
    log = str(tmp_path / "logs" / "run")
    prof = rp.RuntimeProfiler(_args(profile_forward=1), path=str(tmp_path), model_name="m", log_path=log)
    prof.set_model_layer_configs([{"hidden_size": 64, "layer_num": 2, "seq_len": 32}])
    prof.set_time_profiler(start_iter=2, end_iter=4, exit=False)
    prof.tokens_per_iter = 256
    for it, dt in enumerate([9.0, 9.0, 0.5, 0.7, 0.4, 0.6]):
        prof.profile_time_start(it)
        clock["t"] += dt
        prof.profile_time_end(it, loss=2.0 - 0.1 * it, learning_rate=1e-4, grad_norm=1.5)
        clock["t"] += 0.05                                     # time outside the bracket is not counted
    # the window [2, 4) was averaged and written, then slid to [4, 6)
    assert json.load(open(prof.time_profiling_path())) == {"layernum[2]_bsz8_seq32": pytest.approx(500.0)}
    assert prof.last_average_time == pytest.approx(0.5) and (prof.start_iter, prof.end_iter) == (6, 8)
    out = capsys.readouterr().out
    assert "Average iteration time is: 0.6000 s" in out and "Average iteration time is: 0.5000 s" in out
    assert "| Iteration:      3 | Consumed samples:           24 | Elapsed time per iteration (ms): 500.0 |" in out
    lines = [json.loads(l) for l in open(log + ".rank0.jsonl")]
    assert len(lines) == 6 and lines[2]["step_time_s_max_over_ranks"] == pytest.approx(0.5)
    assert lines[2]["tokens_per_s"] == pytest.approx(512.0) and lines[3]["loss"] == pytest.approx(1.7)


def test_runtime_profiler_exit_after_window(tmp_path, monkeypatch):
    monkeypatch.setattr(rp.torch.cuda, "is_available", lambda: False)
    prof = rp.RuntimeProfiler(_args(save_profiled_iteration=1), path=str(tmp_path), model_name="m")
    prof.set_model_layer_configs([{"hidden_size": 64, "layer_num": 2, "seq_len": 32}])
    prof.set_time_profiler(start_iter=0, end_iter=2, exit=True)
    prof.profile_time_start(0)
    prof.profile_time_end(0)
    prof.profile_time_start(1)
    with pytest.raises(SystemExit):
        prof.profile_time_end(1)
    assert list(json.load(open(prof.time_profiling_path()))) == ["layernum[2]_bsz8_seq32_iter"]


# ---------------------------------------------------------------------------------------------- hardware profiler
def test_hardware_group_enumeration():
    g = HardwareProfiler.group_ranks
    assert g(8, 8, True) == [list(range(8))]
    assert g(8, 4, True) == [[0, 1, 2, 3], [4, 5, 6, 7]] and g(8, 4, False) == [[0, 2, 4, 6], [1, 3, 5, 7]]
    assert g(8, 2, True) == [[0, 1], [2, 3], [4, 5], [6, 7]] and g(8, 2, False) == [[0, 4], [1, 5], [2, 6], [3, 7]]
    for size in (2, 4, 8):
        for consec in (True, False):
            flat = sorted(r for grp in g(8, size, consec) for r in grp)
            assert flat == list(range(8)) and all(len(grp) == size for grp in g(8, size, consec))


def test_hardware_profiler_files_and_keys(tmp_path, monkeypatch):
    """Every measurement replaced by a canned table: checks file names, keys and that the search readers accept them."""
    from hetu_galvatron_b200.profiler import hardware_profiler as hp
    from hetu_galvatron_b200.utils.config_utils import read_allreduce_bandwidth_config, read_p2p_bandwidth_config, remap_config

    args = SimpleNamespace(num_nodes=1, num_gpus_per_node=8, max_pp_deg=8, start_mb=1, end_mb=1024)
    prof = HardwareProfiler(args)
    prof.set_path(str(tmp_path))
    ar = {"allreduce_size_8_consec_1": 650.0}
    for k in (4, 2):
        for c in (0, 1):
            ar["allreduce_size_%d_consec_%d" % (k, c)] = 600.0 - 10 * k + c
    sp = {}
    for k in (8, 4, 2):
        for mb in (1, 2, 4, 8, 16, 32, 64, 128, 256, 512, 1024):
            sp["allreduce_size_%d_%dMB_time" % (k, mb)] = 0.02 + 0.004 * mb
            sp["all2all_size_%d_%dMB_time" % (k, mb)] = 0.015 + 0.002 * mb
    monkeypatch.setattr(prof, "profile_allreduce_bandwidth", lambda: ar)
    monkeypatch.setattr(prof, "profile_p2p_bandwidth", lambda: {"pp_size_2": 700.0, "pp_size_4": 690.0, "pp_size_8": 680.0})
    monkeypatch.setattr(prof, "profile_sp_time", lambda *a, **k: sp)
    monkeypatch.setattr(prof, "profile_overlap", lambda: {"overlap_coe": 1.12, "compute_ms": 1.0, "comm_ms": 2.0})
    monkeypatch.setattr(prof, "profile_native", lambda: (_ for _ in ()).throw(RuntimeError("no symmetric memory here")))
    monkeypatch.setattr(hp.dist, "get_rank", lambda: 0)
    res = prof.profile_all()
    assert res["native"] == {"unavailable": "no symmetric memory here"}
    d = os.path.join(str(tmp_path), "hardware_configs")
    assert sorted(os.listdir(d)) == ["allreduce_bandwidth_1nodes_8gpus_per_node.json", "nvlink_native_1nodes_8gpus_per_node.json",
                                     "overlap_coefficient.json", "p2p_bandwidth_1nodes_8gpus_per_node.json",
                                     "sp_time_1nodes_8gpus_per_node.json"]
    bw, coe = read_allreduce_bandwidth_config(os.path.join(d, "allreduce_bandwidth_1nodes_8gpus_per_node.json"), 8)
    assert coe["8"] == pytest.approx(1 / 650.0) and bw["4_1"] == 561.0
    p2p, _ = read_p2p_bandwidth_config(os.path.join(d, "p2p_bandwidth_1nodes_8gpus_per_node.json"))
    assert p2p == {2: 700.0, 4: 690.0, 8: 680.0}
    assert json.load(open(os.path.join(d, "overlap_coefficient.json"))) == {"overlap_coe": 1.12}
    table = remap_config(json.load(open(os.path.join(d, "sp_time_1nodes_8gpus_per_node.json"))), "all2all")
    assert sorted(table) == [2, 4, 8] and table[8]["popt"] == pytest.approx([0.002, 0.015], rel=1e-4)


def test_hardware_profiler_launch_command(monkeypatch):
    from hetu_galvatron_b200.profiler import hardware_profiler as hp

    seen = {}
    monkeypatch.setattr(hp.subprocess, "call", lambda cmd: seen.setdefault("cmd", cmd) and 0)
    prof = HardwareProfiler(SimpleNamespace(num_nodes=1, num_gpus_per_node=4))
    assert prof.launch("x.py", ["--flag", "1"]) == 0
    cmd = seen["cmd"]
    assert cmd[1:4] == ["-m", "torch.distributed.run", "--nnodes=1"] and cmd[cmd.index("--nproc-per-node") + 1] == "4"
    assert cmd[cmd.index("--master-addr") + 1] == "127.0.0.1" and cmd[-3:] == ["x.py", "--flag", "1"]


def test_hardware_profiler_single_table_selection(tmp_path, monkeypatch):
    from hetu_galvatron_b200.profiler import hardware_profiler as hp

    prof = HardwareProfiler(SimpleNamespace(num_nodes=1, num_gpus_per_node=8, max_pp_deg=8, start_mb=1, end_mb=1024))
    prof.set_path(str(tmp_path))
    called = []
    monkeypatch.setattr(prof, "profile_allreduce_bandwidth", lambda: called.append("allreduce") or {"allreduce_size_8_consec_1": 1.0})
    monkeypatch.setattr(prof, "profile_p2p_bandwidth", lambda: called.append("p2p") or {"pp_size_2": 1.0})
    monkeypatch.setattr(prof, "profile_sp_time", lambda *a, **k: called.append("sp") or {})
    monkeypatch.setattr(prof, "profile_overlap", lambda: called.append("overlap") or {"overlap_coe": 1.05, "compute_ms": 1.0})
    monkeypatch.setattr(hp.dist, "get_rank", lambda: 0)
    res = prof.profile_all(only=["overlap"])
    assert called == ["overlap"] and list(res) == ["overlap"]
    assert os.listdir(os.path.join(str(tmp_path), "hardware_configs")) == ["overlap_coefficient.json"]
    res = prof.profile_all(only=["p2p", "allreduce"])
    assert sorted(called[1:]) == ["allreduce", "p2p"] and sorted(res) == ["allreduce", "p2p"]
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(hp.__file__))), "profile_hardware")
    for name in ("profile_hardware", "profile_allreduce", "profile_p2p", "profile_all2all", "profile_overlap"):
        assert os.path.exists(os.path.join(root, name + ".py"))
