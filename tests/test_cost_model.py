"""Closed-form checks of the memory / time / other-time cost models on hand-made profiles (the reference checks the
same properties in tests/search_engine/test_cost_model.py:19-630). CPU only; nothing here touches torch."""
import numpy as np
import pytest

from hetu_galvatron_b200.search.cost_model import (MemoryCostModel, OtherTimeCostModel, TimeCostModel, chunk_like_torch,
                                                   get_real_chunk, get_time_cost_all_stages)
from hetu_galvatron_b200.search.cost_model_args import ModelArgs, ParallelArgs, ProfileHardwareArgs, ProfileModelArgs, TrainArgs

ACT = {1: 85.0, 2: 47.0, 4: 28.0, 8: 18.5, "checkpoint": 10.0}
OTHER_OFF = {"model_states": {1: 640.0, 2: 320.0, 4: 160.0, 8: 80.0}, "activation": {1: 320.0, 2: 160.0, 4: 80.0, 8: 40.0}}
OTHER_ON = {"first_stage": {"model_states": {1: 400.0, 2: 200.0, 4: 100.0, 8: 50.0}, "activation": {1: 100.0, 2: 50.0, 4: 25.0, 8: 12.5}},
            "last_stage": {"model_states": {1: 240.0, 2: 120.0, 4: 60.0, 8: 30.0}, "activation": {1: 220.0, 2: 110.0, 4: 55.0, 8: 27.5}}}


def memory_model(strategy, gbs=32, chunks=4, stage_idx=0, vsp=0, embed_sdp=False, **over):
    train = TrainArgs(mixed_precision=over.pop("mixed_precision", True), async_grad_reduce=over.pop("async_grad_reduce", True),
                      pytorch_context_mem=over.pop("pytorch_context_mem", 1024),
                      memory_layout=over.pop("memory_layout", "fsdp"), grad_bytes=over.pop("grad_bytes", 4),
                      fused_engine=over.pop("fused_engine", False))
    par = ParallelArgs(use_zero2_for_dp=over.pop("use_zero2_for_dp", False), disable_vtp=over.pop("disable_vtp", False),
                       sequence_parallel=over.pop("sequence_parallel", True), pipeline_type=over.pop("pipeline_type", "gpipe"),
                       chunks=chunks)
    par.max_tp_deg = 8
    prof = ProfileModelArgs(tp_activation_per_bsz_dict=dict(ACT), other_memory_pp_off=OTHER_OFF, other_memory_pp_on=OTHER_ON)
    assert not over, over
    return MemoryCostModel(strategy, global_batch_size=gbs, mbsz=2, min_tp=1, max_tp=8, stage_idx=stage_idx, vsp=vsp,
                           embed_sdp=embed_sdp, model_args=ModelArgs(parameter_size=48), train_args=train, parallel_args=par,
                           profile_model_args=prof)


def test_chunking_follows_torch_chunk():
    assert [len(b) for b in chunk_like_torch(10, 4)] == [3, 3, 3, 1]
    assert [len(b) for b in chunk_like_torch(8, 3)] == [3, 3, 2]
    assert get_real_chunk(6, 4) == 3 and get_real_chunk(5, 1) == 1 and get_real_chunk(8, 8) == 8
    with pytest.raises(ValueError):
        chunk_like_torch(4, 0)


def test_memory_pure_dp():
    m = memory_model([1, 1, 8, {"fsdp": 0}], gbs=32, chunks=1)
    c = m.get_memory_cost()
    assert m.sdp_size == 8 and c["parameter"] == 48 and c["model_states"] == 4 * 48
    assert c["activation"] == pytest.approx(ACT[1] * 32 / 8)
    assert c["enc_total"] == pytest.approx(c["model_states"] + c["activation"])
    # pp off: candidates 1..8, each one stage holding embedding + head + context
    assert sorted(c["other"]) == [1, 2, 4, 8]
    for tp, stages in c["other"].items():
        assert len(stages) == 1
        assert stages[0] == pytest.approx(OTHER_OFF["model_states"][tp] + OTHER_OFF["activation"][tp] * 32 * tp / 8 + 1024)


def test_memory_tp_and_checkpoint_under_sequence_parallel():
    c = memory_model([1, 2, 4, {"fsdp": 0, "cpt": 1}], chunks=1).get_memory_cost()
    assert c["parameter"] == 24 and c["model_states"] == 96
    assert c["activation"] == pytest.approx(ACT["checkpoint"] * 8 / 2)            # boundary activation split over tp
    c2 = memory_model([1, 2, 4, {"fsdp": 0, "cpt": 1}], chunks=1, sequence_parallel=False).get_memory_cost()
    assert c2["activation"] == pytest.approx(ACT["checkpoint"] * 8)
    c3 = memory_model([1, 2, 4, {"fsdp": 0}], chunks=1).get_memory_cost()
    assert c3["activation"] == pytest.approx(ACT[2] * 8)


def test_memory_ulysses_replicates_weights_and_shards_over_tp_times_dp():
    m = memory_model([1, 4, 2, {"sp": 1, "fsdp": 1}], chunks=1)
    assert m.sdp_size == 8 and m.parameter_size == 48
    assert m.model_states_size == pytest.approx(4 * 48 * (1 / 8 + 0.003))
    m = memory_model([1, 4, 2, {"fsdp": 1}], chunks=1)
    assert m.sdp_size == 2 and m.parameter_size == 12
    assert m.model_states_size == pytest.approx(4 * 12 * (1 / 2 + 0.003))


@pytest.mark.parametrize("chunks,mixed,async_reduce,z2,z3", [
    (1, True, True, lambda s: 7 / 8 * s + 1 / 8, lambda s: s),
    (1, False, True, lambda s: 3 / 4 * s + 1 / 4, lambda s: s),
    (4, True, True, lambda s: 6 / 8 * s + 2 / 8, lambda s: 7 / 8 * s + 1 / 8),
    (4, False, True, lambda s: 2 / 4 * s + 2 / 4, lambda s: 3 / 4 * s + 1 / 4),
    (4, True, False, lambda s: (7 / 8 * s + 1 / 8) * 5 / 4, lambda s: s * 5 / 4),
])
def test_memory_zero_ratios(chunks, mixed, async_reduce, z2, z3):
    shard = 1 / 4 + 0.003
    kw = dict(gbs=32, chunks=chunks, mixed_precision=mixed, async_grad_reduce=async_reduce)
    m2 = memory_model([1, 2, 4, {"fsdp": 0}], use_zero2_for_dp=True, **kw)
    m3 = memory_model([1, 2, 4, {"fsdp": 1}], **kw)
    ddp = memory_model([1, 2, 4, {"fsdp": 0}], **kw)
    assert ddp.model_states_size == pytest.approx(96)
    assert m2.model_states_size == pytest.approx(96 * z2(shard))
    assert m3.model_states_size == pytest.approx(96 * z3(shard))
    assert m3.model_states_size <= m2.model_states_size <= ddp.model_states_size * 1.25 + 1e-9


def test_engine_layout_counts_what_the_zero_engine_keeps():
    """16 bytes per parameter = 4 x parameter_size. Mixed precision: 2 (bf16 copy) + gradient buffer + 12 (master and two
    moments); the gradient buffer is never sharded, ZeRO-2 shards the 12, ZeRO-3 the 2 as well."""
    from hetu_galvatron_b200.search.cost_model import engine_state_ratio as r

    assert r("ddp", 8, True, 4) == pytest.approx(18 / 16) and r("ddp", 8, True, 2) == pytest.approx(1.0)
    assert r("zero2", 8, True, 2) == pytest.approx((4 + 12 / 8) / 16)
    assert r("zero3", 4, True, 4) == pytest.approx((4 + 14 / 4) / 16)
    assert r("zero3", 2, True, 4, settled=True) == pytest.approx(13 / 16)      # + the fp32 reduced slice after an iteration
    assert r("zero2", 1, True, 4) == r("ddp", 1, True, 4) == r("zero3", 1, True, 4)
    assert r("ddp", 4, False, 4) == pytest.approx(1.0) and r("zero2", 4, False, 4) == pytest.approx((8 + 8 / 4) / 16)
    with pytest.raises(ValueError):
        r("zero1", 2, True, 4)
    kw = dict(gbs=32, chunks=4, memory_layout="engine", grad_bytes=2)
    ddp = memory_model([1, 2, 4, {"fsdp": 0}], **kw)
    m2 = memory_model([1, 2, 4, {"fsdp": 0}], use_zero2_for_dp=True, **kw)
    m3 = memory_model([1, 2, 4, {"fsdp": 1}], **kw)
    assert ddp.model_states_size == pytest.approx(96) and m2.model_states_size == pytest.approx(96 * (4 + 3) / 16)
    assert m3.model_states_size == pytest.approx(96 * (2 + 14 / 4) / 16)
    # embedding / head follow the same layout
    off = OTHER_OFF["model_states"][1]
    assert m2.other_memory_cost[1][0] - ddp.other_memory_cost[1][0] == pytest.approx(off * ((4 + 12 / 8) / 16 - 1.0))
    # the peer-memory engine keeps its fp32 reduced slice for the whole run: 4 more bytes per parameter over the sharding degree
    f2 = memory_model([1, 2, 4, {"fsdp": 0}], use_zero2_for_dp=True, fused_engine=True, **kw)
    assert f2.model_states_size == pytest.approx(96 * (4 + (12 + 4) / 4) / 16)
    assert memory_model([1, 2, 4, {"fsdp": 0}], fused_engine=True, **kw).model_states_size == pytest.approx(ddp.model_states_size)
    # chunk count and asynchronous reduction do not change what the engine keeps
    assert memory_model([1, 2, 4, {"fsdp": 1}], gbs=32, chunks=1, memory_layout="engine", grad_bytes=2,
                        async_grad_reduce=False).model_states_size == pytest.approx(m3.model_states_size)


def test_memory_1f1b_keeps_fewer_microbatches_on_later_stages():
    first = memory_model([4, 1, 2, {"fsdp": 0}], gbs=32, chunks=8, stage_idx=0, pipeline_type="pipedream_flush")
    last = memory_model([4, 1, 2, {"fsdp": 0}], gbs=32, chunks=8, stage_idx=3, pipeline_type="pipedream_flush")
    gpipe = memory_model([4, 1, 2, {"fsdp": 0}], gbs=32, chunks=8, stage_idx=0, pipeline_type="gpipe")
    assert first.act_1f1b_ratio == pytest.approx(4 / 8) and last.act_1f1b_ratio == pytest.approx(1 / 8)
    assert first.activation_size == pytest.approx(ACT[1] * 16 * 4 / 8)
    assert last.activation_size == pytest.approx(ACT[1] * 16 * 1 / 8)
    assert gpipe.activation_size == pytest.approx(ACT[1] * 2)                 # the DP keeps one micro-batch and scales later
    # embedding on the first stage sees pp micro-batches under 1F1B, the head one
    o = first.other_memory_cost[1]
    bsz = 32 * 1 / 1 / 2 / 8
    assert len(o) == 4 and o[1] == o[2] == 1024
    assert o[0] == pytest.approx(OTHER_ON["first_stage"]["model_states"][1] + OTHER_ON["first_stage"]["activation"][1] * bsz * 4 + 1024)
    assert o[3] == pytest.approx(OTHER_ON["last_stage"]["model_states"][1] + OTHER_ON["last_stage"]["activation"][1] * bsz + 1024)


def test_memory_other_with_vsp_and_embed_sdp():
    plain = memory_model([1, 4, 2, {"fsdp": 0}], chunks=1)
    vsp = memory_model([1, 4, 2, {"fsdp": 0}], chunks=1, vsp=1)
    esdp = memory_model([1, 4, 2, {"fsdp": 0}], chunks=1, embed_sdp=True)
    off = OTHER_OFF
    act = lambda tp: off["activation"][tp] * 32 * tp / 4 / 2
    assert plain.other_memory_cost[4][0] == pytest.approx(off["model_states"][4] + act(4) + 1024)
    assert vsp.other_memory_cost[4][0] == pytest.approx(off["model_states"][1] + act(4) + 1024)      # replicated vocab
    assert esdp.other_memory_cost[4][0] == pytest.approx(off["model_states"][4] * (1 / 2 + 0.003) + act(4) + 1024)
    assert list(memory_model([1, 4, 2, {"fsdp": 0}], chunks=1, disable_vtp=True).other_memory_cost) == [1]


# ---------------------------------------------------------------------------------------------- time
SP_TABLE = {2: {"popt": np.array([0.01, 0.05])}, 4: {"popt": np.array([0.012, 0.06])}, 8: {"popt": np.array([0.015, 0.08])}}
A2A_TABLE = {2: {"popt": np.array([0.005, 0.03])}, 4: {"popt": np.array([0.006, 0.04])}, 8: {"popt": np.array([0.008, 0.05])}}


def time_model(strategy, gbs=32, sp_space="tp", fct=2.0, hw=None, **over):
    hw = hw or ProfileHardwareArgs(allreduce_dict=SP_TABLE, all2all_dict=A2A_TABLE)
    return TimeCostModel(strategy, global_batch_size=gbs, no_comm=over.pop("no_comm", False),
                         model_args=ModelArgs(parameter_size=48, seq_length=1024, hidden_size=4096, layer_num=16),
                         train_args=TrainArgs(mixed_precision=over.pop("mixed_precision", True)),
                         parallel_args=ParallelArgs(sp_space=sp_space, use_zero2_for_dp=over.pop("use_zero2_for_dp", False)),
                         profile_model_args=ProfileModelArgs(forward_computation_time=fct, optimizer_time=over.pop("optimizer_time", 0.0)),
                         profile_hardware_args=hw, **over)


def test_time_single_gpu_is_forward_plus_backward():
    m = time_model([1, 1, 1, {}], gbs=8)
    assert m.fct == pytest.approx(2.0 * 8 * 16) and m.bct == pytest.approx(2 * m.fct)
    assert m.gen_result() == pytest.approx((m.fct + m.bct) * 0.001 / 16)
    ck = time_model([1, 1, 1, {"cpt": 1}], gbs=8)
    assert ck.bct == pytest.approx(3 * ck.fct)
    assert ck.gen_result() == pytest.approx(4 * ck.fct * 0.001 / 16)


def test_time_optimizer_step_is_paid_once_per_step_and_sharded():
    base = time_model([1, 1, 1, {}], gbs=8).gen_result()
    m = time_model([1, 1, 1, {}], gbs=8, optimizer_time=1.2)
    assert m.optimizer_ms() == pytest.approx(1.2) and m.gen_result() == pytest.approx(base + 1.2e-3)
    assert time_model([1, 1, 1, {}], gbs=8, optimizer_time=1.2, with_optimizer=False).gen_result() == pytest.approx(base)
    assert time_model([1, 2, 4, {"tp": 1, "fsdp": 0}], optimizer_time=1.2).optimizer_ms() == pytest.approx(0.6)          # DDP: every replica steps
    assert time_model([1, 2, 4, {"tp": 1, "fsdp": 0}], optimizer_time=1.2, use_zero2_for_dp=True).optimizer_ms() == pytest.approx(0.6 / 4)
    assert time_model([1, 2, 4, {"tp": 1, "fsdp": 1}], optimizer_time=1.2).optimizer_ms() == pytest.approx(0.6 / 4)
    assert time_model([1, 4, 2, {"tp": 1, "sp": 1, "fsdp": 1}], sp_space="tp+sp", optimizer_time=1.2).optimizer_ms() == pytest.approx(1.2 / 8)   # Ulysses: weights whole, 8 shards
    # the pipelined composition counts it once whatever the number of micro-batches
    hw = ProfileHardwareArgs(allreduce_dict=SP_TABLE, all2all_dict=A2A_TABLE)
    args = dict(layer_num_list=[16], model_args_list=[ModelArgs(parameter_size=48, seq_length=1024, hidden_size=4096, layer_num=16)],
                train_args_list=[TrainArgs(mixed_precision=True)], parallel_args_list=[ParallelArgs(sp_space="tp")],
                profile_hardware_args_list=[hw], strategies=[[1, 1, 1, {}]] * 16, partition=[16], bsz=8, min_tp=1, other_time_cost=[0.0])
    from hetu_galvatron_b200.search.cost_model import pipeline_costmodel
    for chunks in (1, 4):
        plain = pipeline_costmodel(TimeCostModel, profile_model_args_list=[ProfileModelArgs(forward_computation_time=2.0)], chunks=chunks, **args)
        timed = pipeline_costmodel(TimeCostModel, profile_model_args_list=[ProfileModelArgs(forward_computation_time=2.0, optimizer_time=1.2)],
                                   chunks=chunks, **args)
        assert timed - plain == pytest.approx(16 * 1.2e-3)


def test_time_forward_profile_as_fitted_line():
    m = time_model([1, 2, 4, {"tp": 1}], gbs=32, fct=np.array([1.5, 0.25]))
    assert m.fct == pytest.approx((1.5 * (32 / 4 / 2) + 0.25) * 16)


def test_time_dp_overlap_is_piecewise_and_continuous():
    m = time_model([1, 1, 8, {"fsdp": 0}], gbs=64)
    assert m.dp_message_size == pytest.approx(2 * 7 / 8 * 48 * 16 / 2)
    assert m.dc == pytest.approx(ProfileHardwareArgs().comm_coe_dict["8"]) and m.dc_overlap == pytest.approx(1.3 * m.dc)
    # compute-bound: all communication hides, what is left of the backward runs at full speed
    over, rest, _ = m.bct_dp_overlap(100.0, 1000.0)
    assert over == pytest.approx(100 * m.dc_overlap) and rest == pytest.approx(1000 - over / 1.3)
    # communication-bound
    over, rest, _ = m.bct_dp_overlap(1e6, 10.0)
    assert over == pytest.approx(13.0) and rest == pytest.approx((1e6 - 13.0 / m.dc_overlap) * m.dc)
    # at the crossing point both branches agree
    x = 10.0 * 1.3 / m.dc_overlap
    lo, hi = m.bct_dp_overlap(x * (1 - 1e-9), 10.0), m.bct_dp_overlap(x * (1 + 1e-9), 10.0)
    assert lo[0] + lo[1] == pytest.approx(hi[0] + hi[1], rel=1e-6)
    over, rest, _ = m.bct_dp_overlap(m.dp_message_size, m.bct)
    assert m.gen_result() == pytest.approx((m.fct + over + rest) * 0.001 / 16)
    assert time_model([1, 1, 8, {"fsdp": 0}], gbs=64, no_comm=True).dp_message_size == 0


def test_time_tensor_parallel_traffic_both_models():
    # additive bandwidth model: 4 all-reduces of b*s*h per layer, (t-1)/t on the wire
    m = time_model([1, 4, 1, {"tp": 1}], gbs=8, sp_space="tp")
    size = 2 * 3 / 4 * (8 * 1024 * 4096 * 4 * 4 / 2 ** 20) * 16 / 2
    assert m.tp_message_size == pytest.approx(size)
    assert m.tp_communication_time == pytest.approx(size * ProfileHardwareArgs().comm_coe_dict["4_1"])
    assert m.gen_result() == pytest.approx((m.fct + m.bct + m.tp_communication_time) * 0.001 / 16)
    assert time_model([1, 4, 1, {"tp": 1, "cpt": 1}], gbs=8).tp_message_size == pytest.approx(1.5 * size)
    # latency-table model: per-message time from the fitted line of that group size
    s = time_model([1, 4, 1, {"tp": 1}], gbs=8, sp_space="tp+sp")
    mb = 8 * 1024 * 4096 * 2 / 2 ** 20
    assert s.tp_communication_time == pytest.approx(4 * 16 * (0.012 * mb + 0.06))
    u = time_model([1, 4, 1, {"tp": 1, "sp": 1}], gbs=8, sp_space="tp+sp")
    assert u.tp_communication_time == pytest.approx(4 * 16 * (0.006 * mb + 0.04))
    assert u.parameter_size == 48 and u.sdp_size == 4
    # a measured message size is used as is
    hw = ProfileHardwareArgs(allreduce_dict={4: {"popt": np.array([0.012, 0.06]), 8 * 1024 * 4096 * 2: 0.777}}, all2all_dict=A2A_TABLE)
    assert time_model([1, 4, 1, {"tp": 1}], gbs=8, sp_space="tp+sp", hw=hw).tp_communication_time == pytest.approx(64 * 0.777)


def test_time_fused_runtime_scales_only_the_tensor_parallel_term():
    base = time_model([1, 2, 4, {"tp": 1, "fsdp": 0}])
    fused = time_model([1, 2, 4, {"tp": 1, "fsdp": 0}], hw=ProfileHardwareArgs(allreduce_dict=SP_TABLE, all2all_dict=A2A_TABLE,
                                                                               fused_comm_exposed=0.25))
    assert fused.tp_communication_time == pytest.approx(0.25 * base.tp_communication_time)
    assert (base.gen_result() - fused.gen_result()) * 16 / 0.001 == pytest.approx(0.75 * base.tp_communication_time)


def test_time_hybrid_branches_zero3_and_pipeline_terms():
    few_tp = time_model([1, 2, 4, {"tp": 1, "fsdp": 0}])          # tp < world/2: whole backward overlaps
    over, rest, _ = few_tp.bct_dp_overlap(few_tp.dp_message_size, few_tp.bct)
    assert few_tp.gen_result() == pytest.approx((few_tp.fct + over + rest + few_tp.tp_communication_time) * 0.001 / 16)
    assert few_tp.dc == pytest.approx(ProfileHardwareArgs().comm_coe_dict["4_0"])
    many_tp = time_model([1, 4, 2, {"tp": 1, "fsdp": 0}])         # tp >= world/2: half of it
    over, rest, _ = many_tp.bct_dp_overlap(many_tp.dp_message_size, many_tp.bct / 2)
    assert many_tp.gen_result() == pytest.approx((many_tp.fct + many_tp.bct / 2 + over + rest + many_tp.tp_communication_time) * 0.001 / 16)
    z3 = time_model([1, 2, 4, {"tp": 1, "fsdp": 1}])
    assert (z3.gen_result() - few_tp.gen_result()) * 16 / 0.001 == pytest.approx(0.5 * z3.dp_message_size * z3.dc)
    pp = time_model([2, 1, 4, {"fsdp": 0}])
    flat = time_model([1, 1, 4, {"fsdp": 0}])
    msg = 2 * 2 * (32 / 4) * 1024 * 4096 * 4 / 2 ** 20 / 2
    assert pp.p2p_message_size == pytest.approx(msg)
    assert (pp.gen_result() - flat.gen_result()) * 16 / 0.001 == pytest.approx(msg * ProfileHardwareArgs().p2p_comm_coe_dict[2])


# ---------------------------------------------------------------------------------------------- other time
def other_model(pp_deg=1, vsp=False, embed_sdp=False, sp_space="tp", seqs=(1024,), other_time=3.0, min_tp=1, max_tp=8):
    return OtherTimeCostModel(mbsz=4, pp_deg=pp_deg, world_size=8, vsp=vsp, embed_sdp=embed_sdp, min_tp=min_tp, max_tp=max_tp,
                              sequence_length_list=list(seqs), model_args=ModelArgs(hidden_size=4096),
                              train_args=TrainArgs(mixed_precision=True), parallel_args=ParallelArgs(sp_space=sp_space),
                              profile_model_args=ProfileModelArgs(other_memory_pp_off=OTHER_OFF, other_memory_pp_on=OTHER_ON,
                                                                  other_time_profiled=other_time),
                              profile_hardware_args=ProfileHardwareArgs(allreduce_dict=SP_TABLE))


def test_other_time_single_stage():
    m = other_model()
    assert sorted(m.fct) == [1, 2, 4, 8] and m.fct[2] == pytest.approx(4 * 3.0)
    coe = ProfileHardwareArgs().comm_coe_dict
    assert m.dp_size[2] == pytest.approx(OTHER_OFF["model_states"][2] / 4)
    assert m.dp_coe[2] == pytest.approx(coe["4_0"] * 3 / 4) and m.dp_coe[8] == 0 and m.dp_coe[1] == pytest.approx(coe["8"] * 7 / 8)
    one = (2 - 1) / 2 * (4 * 1024 * 4096 / 2 ** 20) * 2 * coe["2_0"]
    assert m.tp_time[2] == pytest.approx(2 * one)                                 # embedding + head
    with_comm, compute_only = m.gen_result()
    grad = m.dp_size[2] * m.dp_coe[2]
    expect = m.get_overlap_time(0.0, 12.0, 0.5 * grad, 24.0, m.tp_time[2]) * 0.001
    assert with_comm[2] == [pytest.approx(expect)]
    assert compute_only[2][0] <= with_comm[2][0]
    assert (m.fwd_factor, m.bwd_factor) == (0.0, 0.5)
    assert (other_model(embed_sdp=True).fwd_factor, other_model(embed_sdp=True).bwd_factor) == (0.5, 1.0)


def test_other_time_pipeline_vsp_and_table_model():
    m = other_model(pp_deg=2)
    assert sorted(m.fct) == [1, 2, 4] and m.fct[1] == (pytest.approx(6.0), pytest.approx(6.0))
    assert m.dp_size[4] == (pytest.approx(25.0), pytest.approx(25.0))             # first-stage table without vsp
    with_comm, _ = m.gen_result()
    assert len(with_comm[1]) == 2 and with_comm[1][0] > 0 and with_comm[1][1] > 0
    v = other_model(pp_deg=2, vsp=True)
    assert v.tp_time[4] == (0, 0) and v.dp_size[4] == (pytest.approx(60.0), pytest.approx(60.0))
    assert v.dp_coe[4] == pytest.approx(ProfileHardwareArgs().comm_coe_dict["4_1"] * 3 / 4)
    s = other_model(sp_space="tp+sp", seqs=(512, 2048))
    mb = lambda seq: 4 * seq * 4096 * 2 / 2 ** 20
    t512, t2048 = 0.01 * mb(512) + 0.05, 0.01 * mb(2048) + 0.05
    assert s.tp_time[2] == pytest.approx(t512 + t2048 + t2048) and s.tp_time[1] == 0
    line = other_model(other_time=np.array([2.0, 0.5]), min_tp=2)
    assert sorted(line.fct) == [2, 4, 8] and line.fct[2] == pytest.approx(2.0 * 2 + 0.5)


def test_overlap_time_phases():
    m = other_model()
    # communication hidden: compute stretched by the overlap coefficient only while the transfer lasts
    assert m.get_overlap_time(1.0, 10.0, 2.0, 20.0, 0.5) == pytest.approx((1 + (13 - 1) / 1.3) + (2 + (26 - 2) / 1.3) + 0.5)
    # communication-bound phases cost the communication time
    assert m.get_overlap_time(50.0, 10.0, 60.0, 20.0, 0.0) == pytest.approx(110.0)


def test_stage_sums():
    assert get_time_cost_all_stages(np.array([1.0, 2.0, 3.0, 4.0, 5.0]), [2, 3]) == [pytest.approx(3.0), pytest.approx(12.0)]
    with pytest.raises(AssertionError):
        get_time_cost_all_stages(np.ones(4), [2, 3])


def test_context_parallel_ranks_extend_the_data_parallel_group():
    """cp_size multiplies the ranks ZeRO shards over and the gradient-reduction group (an extension of the reference)."""
    par = ParallelArgs(chunks=1, sequence_parallel=True, cp_size=2)
    par.max_tp_deg = 8
    prof = ProfileModelArgs(tp_activation_per_bsz_dict=dict(ACT), other_memory_pp_off=OTHER_OFF, other_memory_pp_on=OTHER_ON)
    m = MemoryCostModel([1, 2, 2, {"fsdp": 1}], global_batch_size=8, mbsz=2, min_tp=1, max_tp=8, model_args=ModelArgs(parameter_size=48),
                        train_args=TrainArgs(mixed_precision=True), parallel_args=par, profile_model_args=prof)
    assert m.sdp_size == 4 and m.model_states_size == pytest.approx(96 * (1 / 4 + 0.003))
    hw = ProfileHardwareArgs(allreduce_dict=SP_TABLE, all2all_dict=A2A_TABLE)
    t = TimeCostModel([1, 1, 2, {"fsdp": 0}], global_batch_size=8, model_args=ModelArgs(parameter_size=48, layer_num=16),
                      train_args=TrainArgs(mixed_precision=True), parallel_args=ParallelArgs(sp_space="tp", cp_size=2),
                      profile_model_args=ProfileModelArgs(forward_computation_time=2.0), profile_hardware_args=hw)
    assert t.dp_message_size == pytest.approx(2 * 3 / 4 * 48 * 16 / 2) and t.dc == pytest.approx(hw.comm_coe_dict["4_0"])
    alone = TimeCostModel([1, 1, 1, {}], global_batch_size=8, model_args=ModelArgs(parameter_size=48, layer_num=16),
                          train_args=TrainArgs(mixed_precision=True), parallel_args=ParallelArgs(sp_space="tp", cp_size=2),
                          profile_model_args=ProfileModelArgs(forward_computation_time=2.0), profile_hardware_args=hw)
    over, rest, _ = alone.bct_dp_overlap(alone.dp_message_size, alone.bct)
    assert alone.dp_message_size > 0 and alone.gen_result() == pytest.approx((alone.fct + over + rest) * 0.001 / 16)
