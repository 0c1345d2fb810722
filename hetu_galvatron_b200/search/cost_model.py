"""Memory / time cost models of the strategy search.

What is modelled is the reference's (galvatron/core/search_engine/cost_model.py): per-layer memory =
model states (ZeRO ratios :99-110) + activations (:128-137) and the per-stage "other" memory of embedding and
head (:140-210); per-layer time = forward + backward compute with data-parallel gradient traffic partly
overlapped with the backward pass (:414-431), tensor/sequence-parallel traffic (:345-403), ZeRO-3 gathers and
pipeline p2p (:405-412, :433-466); "other" time of embedding/head (:468-658); and the pipeline composition
(:695-768). The arithmetic is organised as small pure functions over the strategy; the classes are thin
views that keep the reference's constructor signatures and result accessors, because the DP driver and
user code call them by those names.

Extensions: ``ProfileHardwareArgs.fused_comm_exposed`` scales the tensor/sequence-parallel communication
term, for runtimes whose collectives are fused into the neighbouring GEMM and mostly hidden behind it; and
``TrainArgs.memory_layout = "engine"`` prices model states with what this package's ZeRO engine really keeps per rank
(``engine_state_ratio``) instead of the reference's FSDP ratios.
"""
from __future__ import annotations

from types import SimpleNamespace
from typing import List

import numpy as np

from .cost_model_args import ModelArgs, ParallelArgs, ProfileHardwareArgs, ProfileModelArgs, TrainArgs


# ------------------------------------------------------------------------------------------ helpers
def chunk_like_torch(size: int, chunks: int):
    """Index blocks of ``torch.arange(size).chunk(chunks)``: ceil-sized blocks, possibly fewer than ``chunks``."""
    if chunks <= 0:
        raise ValueError("chunks must be positive")
    step = -(-size // chunks)
    return [np.arange(lo, min(lo + step, size)) for lo in range(0, size, step)] if step > 0 else []


def get_real_chunk(local_bsz, chunk) -> int:
    if chunk == 1:
        return 1
    return len(chunk_like_torch(int(local_bsz), int(chunk)))


def _flag(strategy, key) -> bool:
    return bool(strategy[-1].get(key, 0))


def _coe(comm_coe_dict: dict, size: int, variant: str = "") -> float:
    """Communication coefficient (ms/MB) of a group of ``size`` ranks; ``variant`` is '', '_0' or '_1'."""
    if variant == "":
        key = "%d" % size
        return comm_coe_dict[key] if key in comm_coe_dict else comm_coe_dict["%d_1" % size]
    return comm_coe_dict["%d%s" % (size, variant)]


def _coe_any(comm_coe_dict: dict, size: int, variant: str) -> float:
    """Coefficient of a group of ``size`` ranks, preferring ``variant`` and falling back to whichever form the table has."""
    for key in ("%d%s" % (size, variant), "%d" % size, "%d_1" % size, "%d_0" % size):
        if key in comm_coe_dict:
            return comm_coe_dict[key]
    raise KeyError("no bandwidth entry for a group of %d ranks" % size)


def _line(x, popt):
    return popt[0] * x + popt[1]


def _zero_ratios(chunks: int, mixed: bool, async_reduce: bool):
    """(zero2_ratio(d), zero3_ratio(d)): fraction of the 4x-parameter model states a rank keeps."""
    shard = lambda d: 1 / d + 0.003
    if chunks == 1:
        z2 = (lambda d: 7 / 8 * shard(d) + 1 / 8) if mixed else (lambda d: 3 / 4 * shard(d) + 1 / 4)
        return z2, shard
    if async_reduce:
        z2 = (lambda d: 6 / 8 * shard(d) + 2 / 8) if mixed else (lambda d: 2 / 4 * shard(d) + 2 / 4)
        z3 = (lambda d: 7 / 8 * shard(d) + 1 / 8) if mixed else (lambda d: 3 / 4 * shard(d) + 1 / 4)
        return z2, z3
    z2 = (lambda d: (7 / 8 * shard(d) + 1 / 8) * 5 / 4) if mixed else (lambda d: 3 / 4 * shard(d) + 1 / 4)
    return z2, (lambda d: shard(d) * 5 / 4)


def engine_state_ratio(dp_type: str, d: int, mixed: bool, grad_bytes: int = 4, settled: bool = False) -> float:
    """Model states one rank of this package's ZeRO engine (parallel/zero.py) holds, as a fraction of the 16 bytes per
    parameter that ``4 x parameter_size`` stands for.

    Per parameter the engine keeps: the compute-precision copy (2 bytes under mixed precision; in fp32 runs the
    parameters are their own master copy, 4 bytes), a full-size flat gradient buffer of ``grad_bytes`` that lives for
    the whole run whatever the ZeRO stage (micro-batches accumulate into it; under the peer-memory engine it is the
    buffer the other ranks read), and the optimizer slice (fp32 master + two Adam moments = 12 bytes mixed, 8 in fp32).
    ZeRO-2 shards the optimizer slice over ``d`` ranks, ZeRO-3 the parameters too. ``settled`` adds the fp32 reduced
    gradient slice that exists between a bucket's reduction and ``zero_grad``: the state the memory profiler samples
    after an iteration, not the state at the activation peak that the search has to bound."""
    p, opt = (2, 12) if mixed else (4, 8)
    red = 4 if settled else 0
    if dp_type == "ddp" or d <= 1:
        return (p + grad_bytes + opt) / 16
    if dp_type == "zero2":
        return (p + grad_bytes + (opt + red) / d) / 16
    if dp_type == "zero3":
        return (grad_bytes + (p + opt + red) / d) / 16
    raise ValueError("unknown data-parallel type %r" % dp_type)


def _collect(target: SimpleNamespace, wanted: dict, **bundles) -> None:
    for cls_name, bundle in bundles.items():
        for key, value in vars(bundle).items():
            if key in wanted[cls_name]:
                setattr(target, key, value)


# ------------------------------------------------------------------------------------------ memory
class MemoryCostModel:
    memory_args_list = {
        "ModelArgs": ["parameter_size"],
        "TrainArgs": ["mixed_precision", "async_grad_reduce", "pytorch_context_mem", "memory_layout", "grad_bytes", "fused_engine"],
        "ParallelArgs": ["use_zero2_for_dp", "max_tp_deg", "disable_vtp", "sequence_parallel", "sp_space", "pipeline_type",
                         "optimal_chunk_func", "chunks", "cp_size"],
        "ProfileModelArgs": ["tp_activation_per_bsz_dict", "other_memory_pp_off", "other_memory_pp_on"],
    }

    def __init__(self, strategy, global_batch_size: int = 8, mbsz: int = -1, min_tp: int = -1, max_tp: int = -1,
                 stage_idx: int = 0, vsp: int = 0, embed_sdp: bool = False, model_args: ModelArgs = None,
                 train_args: TrainArgs = None, parallel_args: ParallelArgs = None,
                 profile_model_args: ProfileModelArgs = None, logger=None):
        assert mbsz > -1, f"Invalid mbsz: {mbsz}"
        assert min_tp > -1, f"Invalid min_tp: {min_tp}"
        assert all(x is not None for x in (model_args, train_args, parallel_args, profile_model_args)), \
            "One or more variables are None"
        a = self.args = SimpleNamespace(strategy=strategy, global_batch_size=global_batch_size, mbsz=mbsz, min_tp=min_tp,
                                        max_tp=max_tp, stage_idx=stage_idx, vsp=vsp, embed_sdp=embed_sdp)
        self.logger = logger
        _collect(a, self.memory_args_list, ProfileModelArgs=profile_model_args, ModelArgs=model_args, TrainArgs=train_args,
                 ParallelArgs=parallel_args)
        self.pp_size, self.tp_size, self.dp_size = strategy[0], strategy[1], strategy[2]
        ulysses = strategy[-1].get("sp", 0) == 1
        self.sdp_size = (self.tp_size * self.dp_size if ulysses else self.dp_size) * getattr(a, "cp_size", 1)

        # micro-batching: the searched chunk count, capped by what the local batch allows
        if a.chunks is None:
            a.chunks = a.optimal_chunk_func(global_batch_size // self.dp_size, strategy, mbsz, min_tp)
        cap = global_batch_size // (self.tp_size * self.dp_size // min_tp)
        cap = max(cap, 1)
        self.chunks = int(min(a.chunks, cap))
        local = int(global_batch_size / self.dp_size / (self.tp_size // min_tp))
        micro = [len(b) for b in chunk_like_torch(local, self.chunks)]
        self.bsz = global_batch_size / self.dp_size
        if (a.pipeline_type == "pipedream_flush" and self.pp_size > 1) or self.pp_size == 1:
            assert self.chunks == len(micro)
            in_flight = min(self.pp_size - stage_idx, self.chunks)     # micro-batches alive on this stage (1F1B)
            total = np.sum(micro)
            self.act_1f1b_ratio = np.sum(micro[:in_flight]) / total
            self.act_1f1b_ratio_first = np.sum(micro[:min(self.pp_size, self.chunks)]) / total
            self.act_1f1b_ratio_last = micro[0] / total
            self.bsz = self.act_1f1b_ratio * self.bsz
        else:
            self.bsz = micro[0]
        self.engine_layout = getattr(a, "memory_layout", "fsdp") == "engine"
        if self.engine_layout:
            mixed, gb = bool(a.mixed_precision), getattr(a, "grad_bytes", 4)
            keep = bool(getattr(a, "fused_engine", False))       # persistent fp32 reduced slice of the peer-memory engine
            self.ddp_ratio = engine_state_ratio("ddp", 1, mixed, gb)
            self.zero2_ratio = lambda d: engine_state_ratio("zero2", d, mixed, gb, settled=keep)
            self.zero3_ratio = lambda d: engine_state_ratio("zero3", d, mixed, gb, settled=keep)
        else:
            self.ddp_ratio = 1.0
            self.zero2_ratio, self.zero3_ratio = _zero_ratios(self.chunks, a.mixed_precision, a.async_grad_reduce)

        # parameters / model states / activations of one layer
        self.parameter_size = a.parameter_size if ulysses else a.parameter_size / self.tp_size
        self.model_states_size = 4 * self.parameter_size
        if strategy[-1].get("fsdp"):
            self.model_states_size *= self.zero3_ratio(self.sdp_size)
        elif "fsdp" in strategy[-1] and a.use_zero2_for_dp:
            self.model_states_size *= self.zero2_ratio(self.sdp_size)
        else:
            self.model_states_size *= self.ddp_ratio
        if _flag(strategy, "cpt"):
            assert a.tp_activation_per_bsz_dict["checkpoint"] is not None
            self.activation_size = a.tp_activation_per_bsz_dict["checkpoint"] * self.bsz
            if a.sequence_parallel:
                self.activation_size /= self.tp_size
        else:
            self.activation_size = a.tp_activation_per_bsz_dict[self.tp_size] * self.bsz
        self.other_memory_cost = self._other_memory()

    def _other_memory(self) -> dict:
        """Per-stage memory of embedding / head / framework context, for every candidate vocab-tp degree."""
        a = self.args
        if a.disable_vtp:
            candidates = [1]
        else:
            candidates, k = [], a.min_tp
            gpus = a.strategy[0] * a.strategy[1] * a.strategy[2]
            while k * self.pp_size <= gpus and k <= a.max_tp:
                candidates.append(k)
                k *= 2
        off, on = a.other_memory_pp_off, a.other_memory_pp_on
        candidates = [t for t in candidates if t in off["model_states"] and t in on["first_stage"]["model_states"]
                      and t in on["last_stage"]["model_states"]]
        world = self.tp_size * self.dp_size
        out = {}
        for tp in candidates:
            per_stage = [0] * self.pp_size
            bsz = a.global_batch_size * tp / self.tp_size / self.dp_size / self.chunks
            if a.vsp:
                states_tp, shard_over = 1, world
            else:
                states_tp, shard_over = tp, world // tp
            shard_over *= getattr(a, "cp_size", 1)
            if a.embed_sdp:
                ratio = self.zero3_ratio(shard_over)
            elif a.use_zero2_for_dp:
                ratio = self.zero2_ratio(shard_over)
            else:
                ratio = self.ddp_ratio
            if self.pp_size == 1:
                per_stage[0] += off["model_states"][states_tp] * ratio + off["activation"][tp] * bsz
            else:
                first_bsz, last_bsz = (bsz * self.pp_size, bsz) if a.pipeline_type == "pipedream_flush" else (bsz, bsz)
                per_stage[0] += on["first_stage"]["model_states"][states_tp] * ratio + on["first_stage"]["activation"][tp] * first_bsz
                per_stage[-1] += on["last_stage"]["model_states"][states_tp] * ratio + on["last_stage"]["activation"][tp] * last_bsz
            out[tp] = [m + a.pytorch_context_mem for m in per_stage]
        return out

    def get_memory_cost(self) -> dict:
        return {"parameter": self.parameter_size, "model_states": self.model_states_size,
                "activation": self.activation_size, "enc_total": self.model_states_size + self.activation_size,
                "other": self.other_memory_cost}


# ------------------------------------------------------------------------------------------ time
class TimeCostModel:
    time_args_list = {
        "ModelArgs": ["parameter_size", "seq_length", "hidden_size", "layer_num"],
        "TrainArgs": ["mixed_precision", "async_grad_reduce"],
        "ParallelArgs": ["sp_space", "optimal_chunk_func", "cp_size", "use_zero2_for_dp"],
        "ProfileModelArgs": ["forward_computation_time", "optimizer_time"],
        "ProfileHardwareArgs": ["bct_fct_coe", "extra_overhead", "comm_coe_dict", "dp_overlap_coe", "bct_overlap_coe",
                                "p2p_comm_coe_dict", "costmodel_coe", "allreduce_dict", "all2all_dict", "fused_comm_exposed"],
    }

    def __init__(self, strategy, global_batch_size: int = 8, no_comm: bool = False, model_args: ModelArgs = None,
                 train_args: TrainArgs = None, parallel_args: ParallelArgs = None,
                 profile_model_args: ProfileModelArgs = None, profile_hardware_args: ProfileHardwareArgs = None,
                 logger=None, with_optimizer: bool = True):
        assert all(x is not None for x in (model_args, train_args, parallel_args, profile_hardware_args)), \
            "One or more variables are None"
        if model_args.layer_num is None:
            model_args.layer_num = 24
        a = self.args = SimpleNamespace(strategy=strategy, global_batch_size=global_batch_size, no_comm=no_comm,
                                        fused_comm_exposed=1.0, optimizer_time=0.0, use_zero2_for_dp=False)
        self.with_optimizer = with_optimizer
        self.logger = logger
        _collect(a, self.time_args_list, ModelArgs=model_args, TrainArgs=train_args, ParallelArgs=parallel_args,
                 ProfileModelArgs=profile_model_args, ProfileHardwareArgs=profile_hardware_args)
        self.pp_size, self.tp_size, self.dp_size = strategy[0], strategy[1], strategy[2]
        self.sp_space = a.sp_space
        self.fsdp, self.checkpoint = _flag(strategy, "fsdp"), _flag(strategy, "cpt")
        self.ulysses = strategy[-1].get("sp", 0) == 1
        self.sdp_size = self.tp_size * self.dp_size if self.ulysses else self.dp_size
        table = a.all2all_dict if self.ulysses else a.allreduce_dict
        self.sp_dict = np.inf if self.tp_size == 1 else table[self.tp_size]
        self.seq_len, self.hidden_size, self.layer_num = a.seq_length, a.hidden_size, a.layer_num
        self.bsz = global_batch_size / self.dp_size
        self.optimal_microbatch = 1
        self.parameter_size = a.parameter_size if self.ulysses else a.parameter_size / self.tp_size
        self._compute()
        self._dp_comm()
        self._tp_comm()
        self._pp_comm()

    # the consecutive / strided variant named by the strategy's 'tp' flag
    def _variant(self, consecutive_suffix: str, strided_suffix: str) -> str:
        info = self.args.strategy[-1]
        assert "tp" in info and info["tp"] in (0, 1)
        return consecutive_suffix if info["tp"] else strided_suffix

    def _compute(self) -> None:
        a = self.args
        per_rank = self.bsz / self.tp_size
        if isinstance(a.forward_computation_time, np.ndarray):
            self.fct = _line(per_rank, a.forward_computation_time) * self.layer_num
        else:
            self.fct = a.forward_computation_time * self.bsz / self.tp_size * self.layer_num
        self.bct = self.fct * a.bct_fct_coe
        if self.checkpoint:
            self.bct += self.fct

    def _dp_comm(self) -> None:
        a = self.args
        d = self.dp_size * getattr(a, "cp_size", 1)        # gradients are reduced over the context-parallel ranks too
        self.dp_message_size = (2 * (d - 1) / d * self.parameter_size) * self.layer_num
        if a.mixed_precision:
            self.dp_message_size /= 2
        self.fsdp_allgather_message_size = self.dp_message_size * 0.5
        if a.no_comm:
            self.dp_message_size = 0
        cp = getattr(a, "cp_size", 1)
        if cp > 1:
            # the reduction group is cp x dp (x tp under Ulysses) ranks, strided through the machine
            group = (self.sdp_size if self.ulysses else self.dp_size) * cp
            self.dc = _coe_any(a.comm_coe_dict, group, "_0")
        elif self.ulysses:
            self.dc = _coe(a.comm_coe_dict, self.sdp_size)
        elif self.tp_size == 1 or self.dp_size == 1:
            self.dc = _coe(a.comm_coe_dict, self.dp_size)
        else:
            self.dc = _coe(a.comm_coe_dict, self.dp_size, self._variant("_0", "_1"))
        self.dc_overlap = self.dc * a.dp_overlap_coe

    def _tp_comm(self) -> None:
        a = self.args
        elem = 2 if a.mixed_precision else 4
        if self.sp_space == "tp+sp":
            self.tp_comm_num = 4 * self.layer_num
            if self.checkpoint:
                self.tp_comm_num *= 1.5
            if self.tp_size == 1:
                per_message = 0
            else:
                self.per_tp_message_size = self.bsz * self.seq_len * self.hidden_size * elem
                if self.per_tp_message_size in self.sp_dict:
                    per_message = self.sp_dict[self.per_tp_message_size]
                else:
                    per_message = _line(1 / 1024 / 1024 * self.per_tp_message_size, self.sp_dict["popt"])
            self.tp_communication_time = self.tp_comm_num * per_message
        else:
            self.tp_message_size = 2 * (self.tp_size - 1) / self.tp_size * (
                self.bsz * self.seq_len * self.hidden_size * 4 * 4 / 1024 / 1024) * self.layer_num
            if self.checkpoint:
                self.tp_message_size *= 1.5
            if a.mixed_precision:
                self.tp_message_size /= 2
            if self.tp_size == 1 or self.dp_size == 1:
                tc = _coe(a.comm_coe_dict, self.tp_size)
            else:
                tc = _coe(a.comm_coe_dict, self.tp_size, self._variant("_1", "_0"))
            self.tp_communication_time = self.tp_message_size * tc
        self.tp_communication_time *= a.fused_comm_exposed

    def _pp_comm(self) -> None:
        a = self.args
        self.p2p_comm_coe = None
        if self.pp_size > 1 and a.p2p_comm_coe_dict is not None:
            self.p2p_comm_coe = a.p2p_comm_coe_dict[self.pp_size]
            self.p2p_message_size = self.pp_size * 2 * self.bsz * self.seq_len * self.hidden_size * 4 / 1024 / 1024
            if a.mixed_precision:
                self.p2p_message_size = self.p2p_message_size / 2

    def bct_dp_overlap(self, dp_message_size, bct):
        """Backward compute and gradient reduction slow each other down while they overlap; returns the
        overlapped span, what is left of the longer one, and a (always False) 'communication left' flag."""
        a = self.args
        comm = dp_message_size * self.dc_overlap
        comp = bct * a.bct_overlap_coe
        if comm > comp:
            return comp, (dp_message_size - comp / self.dc_overlap) * self.dc, False
        if comm < comp:
            return comm, bct - comm / a.bct_overlap_coe, False
        return comp, 0, False

    def gen_result(self):
        a = self.args
        tp, dp = self.tp_size, self.dp_size * getattr(a, "cp_size", 1)
        if tp == 1 and dp > 1:
            over, rest, _ = self.bct_dp_overlap(self.dp_message_size, self.bct)
            result = self.fct + over + rest + a.extra_overhead
        elif dp == 1 and tp > 1:
            result = self.fct + self.bct + self.tp_communication_time
        elif dp == 1 and tp == 1:
            result = self.fct + self.bct
        elif tp < tp * dp // 2:
            over, rest, _ = self.bct_dp_overlap(self.dp_message_size, self.bct)
            result = self.fct + over + rest + self.tp_communication_time + a.extra_overhead
        else:
            over, rest, _ = self.bct_dp_overlap(self.dp_message_size, self.bct * 1 / 2)
            result = self.fct + 1 / 2 * self.bct + over + rest + self.tp_communication_time + a.extra_overhead
        if self.fsdp:
            result = result + self.fsdp_allgather_message_size * self.dc * self.optimal_microbatch
        if self.pp_size > 1 and self.p2p_comm_coe is not None:
            result = result + self.p2p_message_size * self.p2p_comm_coe
        if self.with_optimizer:
            result = result + self.optimizer_ms() * self.layer_num
        result = result * (0.001 * a.costmodel_coe)
        return result / self.layer_num

    def optimizer_ms(self) -> float:
        """Optimizer step of ONE layer under this strategy, ms per training step: the profiled time of the un-sharded
        layer over the tensor-parallel degree (weights are split) and, under ZeRO-2 / ZeRO-3, over the ranks that share
        the optimizer slice. Paid once per step, not per micro-batch."""
        a = self.args
        t = float(getattr(a, "optimizer_time", 0.0) or 0.0)
        if t <= 0.0:
            return 0.0
        if not self.ulysses:
            t /= self.tp_size
        if self.fsdp or getattr(a, "use_zero2_for_dp", False):
            t /= max(self.sdp_size * getattr(a, "cp_size", 1), 1)
        return t


class OtherTimeCostModel:
    othertime_args_list = {
        "ModelArgs": ["hidden_size"],
        "TrainArgs": ["mixed_precision"],
        "ParallelArgs": ["sp_space"],
        "ProfileModelArgs": ["other_memory_pp_on", "other_memory_pp_off", "other_time_profiled"],
        "ProfileHardwareArgs": ["comm_coe_dict", "allreduce_dict", "dp_overlap_coe", "bct_overlap_coe", "bct_fct_coe"],
    }

    def __init__(self, mbsz: int = 1, pp_deg: int = 2, world_size: int = 8, vsp: bool = False, embed_sdp: bool = False,
                 min_tp: int = 1, max_tp: int = 8, sequence_length_list: list = [512], model_args: ModelArgs = None,
                 train_args: TrainArgs = None, parallel_args: ParallelArgs = None,
                 profile_model_args: ProfileModelArgs = None, profile_hardware_args: ProfileHardwareArgs = None,
                 logger=None):
        assert all(x is not None for x in (model_args, train_args, parallel_args, profile_model_args, profile_hardware_args)), \
            "One or more variables are None"
        a = self.args = SimpleNamespace(mbsz=mbsz, pp_deg=pp_deg, world_size=world_size, vsp=vsp, embed_sdp=embed_sdp,
                                        min_tp=min_tp, max_tp=max_tp, sequence_length_list=sequence_length_list)
        self.logger = logger
        _collect(a, self.othertime_args_list, ModelArgs=model_args, TrainArgs=train_args, ParallelArgs=parallel_args,
                 ProfileModelArgs=profile_model_args, ProfileHardwareArgs=profile_hardware_args)
        self.sequence_length_list, self.hidden_size, self.sp_space = sequence_length_list, a.hidden_size, a.sp_space
        self.dp_coe, self.fct, self.tp_time, self.sp_size, self.dp_size, self.comm_factor = {}, {}, {}, {}, {}, {}
        stage_gpus = world_size // pp_deg
        degrees, k = [], min_tp
        while k <= max_tp and stage_gpus >= k:
            degrees.append(k)
            k *= 2
        for k in degrees:
            self._tp_time(k, stage_gpus)
            self._fct(k)
            self._dp(k, stage_gpus)
        self.fwd_factor, self.bwd_factor = (0.5, 1.0) if embed_sdp else (0.0, 0.5)

    def _tp_time(self, k: int, stage_gpus: int) -> None:
        a = self.args
        elem = 2 if a.mixed_precision else 4
        times = []
        # what the last degree examined moved per sequence length (bytes per all-reduce under "tp+sp", MB otherwise): kept
        # for inspection, as the reference does (cost_model.py:537-563)
        self.per_tp_message_size, self.tp_message_size = [], []
        for seq_len in self.sequence_length_list:
            if a.vsp != 0:
                times.append(0)
            elif self.sp_space == "tp+sp":
                size = a.mbsz * seq_len * a.hidden_size * elem
                self.per_tp_message_size.append(size)
                if k == 1:
                    times.append(0)
                elif size in a.allreduce_dict:
                    times.append(a.allreduce_dict[size])
                else:
                    times.append(_line(1 / 1024 / 1024 * size, a.allreduce_dict[k]["popt"]))
            else:
                dp_size = stage_gpus // k
                tp_coe = _coe(a.comm_coe_dict, k) if (k == 1 or dp_size == 1) else _coe(a.comm_coe_dict, k, "_0")
                self.tp_message_size.append((k - 1) / k * (a.mbsz * seq_len * self.hidden_size / 1024 / 1024) * elem)
                times.append(self.tp_message_size[-1] * tp_coe)
        # embedding at the first sequence length, head at the last (two layer types: encoder-decoder models)
        self.tp_time[k] = (sum(times) + times[-1]) if a.pp_deg == 1 else (times[0], times[-1])

    def _fct(self, k: int) -> None:
        a = self.args
        per = a.mbsz / a.min_tp
        t = _line(per, a.other_time_profiled) if isinstance(a.other_time_profiled, np.ndarray) else per * a.other_time_profiled
        self.fct[k] = t if a.pp_deg == 1 else (t / 2, t / 2)

    def _dp(self, k: int, stage_gpus: int) -> None:
        a = self.args
        if a.vsp == 0:
            dp_size = stage_gpus // k
            coe = _coe(a.comm_coe_dict, dp_size) if (k == 1 or dp_size == 1) else _coe(a.comm_coe_dict, dp_size, "_0")
        else:
            dp_size = stage_gpus
            coe = _coe(a.comm_coe_dict, dp_size)
        self.dp_coe[k] = coe * (dp_size - 1) / dp_size        # bus bandwidth -> algorithm bandwidth
        states_tp = k if a.vsp == 0 else 1
        if a.pp_deg == 1:
            self.dp_size[k] = a.other_memory_pp_off["model_states"][states_tp] / 4
        else:
            stage = "first_stage" if a.vsp == 0 else "last_stage"
            m = a.other_memory_pp_on[stage]["model_states"][states_tp] / 4
            self.dp_size[k] = (m, m)

    def get_overlap_time(self, forward_comm_time, forward_comp_time, backward_comm_time, backward_comp_time, tp_time):
        c = self.args.dp_overlap_coe

        def phase(comm, comp):
            comp = comp * c
            return comm + (comp - comm) / c if comp > comm else comm

        return phase(forward_comm_time, forward_comp_time) + phase(backward_comm_time, backward_comp_time) + tp_time

    def gen_result(self):
        a = self.args
        with_comm, compute_only = {}, {}
        for k in self.dp_size:
            with_comm[k], compute_only[k] = [0] * a.pp_deg, [0] * a.pp_deg
            ends = [(0, None)] if a.pp_deg == 1 else [(0, 0), (-1, -1)]
            for stage, pick in ends:
                size = self.dp_size[k] if pick is None else self.dp_size[k][pick]
                fct = self.fct[k] if pick is None else self.fct[k][pick]
                tp_t = self.tp_time[k] if pick is None else self.tp_time[k][pick]
                grad = size * self.dp_coe[k]
                with_comm[k][stage] = 0.001 * self.get_overlap_time(grad * self.fwd_factor, fct, grad * self.bwd_factor,
                                                                    fct * a.bct_fct_coe, tp_t)
                compute_only[k][stage] = 0.001 * self.get_overlap_time(grad * self.fwd_factor, fct,
                                                                       grad * (self.bwd_factor - 0.5),
                                                                       fct * a.bct_fct_coe, tp_t)
        return with_comm, compute_only


# ------------------------------------------------------------------------------------------ pipeline
def get_time_cost_all_stages(layer_timecosts, pp_stage_division) -> List[float]:
    assert np.sum(pp_stage_division) == len(layer_timecosts)
    bounds = np.concatenate([[0], np.cumsum(pp_stage_division)]).astype(int)
    return [np.sum(layer_timecosts[bounds[i]:bounds[i + 1]]) for i in range(len(pp_stage_division))]


def pipeline_costmodel(timecostmodel, layer_num_list, model_args_list, train_args_list, parallel_args_list,
                       profile_model_args_list, profile_hardware_args_list, strategies, partition, chunks, bsz, min_tp,
                       other_time_cost, logger=None, return_stage_cost: bool = False):
    """Step time of a pipelined plan: per-stage compute of one micro-batch, 1F1B fill/drain with the slowest-first
    assumption, plus the gradient-reduction tail that cannot hide behind the last micro-batches."""
    if strategies is None:
        return ([np.inf] * len(partition), np.inf) if return_stage_cost else np.inf
    from ..utils.strategy_utils import form_strategy, strategy_str2list

    type_of_layer = []
    for t, n in enumerate(layer_num_list):
        type_of_layer += [t] * n
    local = int(bsz / (strategies[0][1] * strategies[0][2] // min_tp))
    if isinstance(chunks, list):
        chunks = [get_real_chunk(local, c) for c in chunks]
        bsz_chunked = [bsz / c for c in chunks]
        max_chunk = np.max(chunks)
    else:
        chunks = get_real_chunk(local, chunks)
        bsz_chunked = [bsz / chunks] * len(layer_num_list)
        max_chunk = chunks
    pp_deg = len(partition)
    names = list(set(form_strategy(s) for s in strategies))
    full, compute, optimizer = {}, {}, {}
    for t in range(len(layer_num_list)):
        kw = dict(model_args=model_args_list[t], train_args=train_args_list[t], parallel_args=parallel_args_list[t],
                  profile_model_args=profile_model_args_list[t], profile_hardware_args=profile_hardware_args_list[t],
                  logger=logger)
        for name in names:
            s = strategy_str2list(name)
            opt_ms = 0.0
            try:
                model = timecostmodel(s, bsz_chunked[t], with_optimizer=False, **kw)
                opt_ms = model.optimizer_ms()
                full[(t, name)] = model.gen_result()
                compute[(t, name)] = timecostmodel(s, bsz_chunked[t], no_comm=True, with_optimizer=False, **kw).gen_result()
            except TypeError:         # a cost-model class without the optimizer term
                full[(t, name)] = timecostmodel(s, bsz_chunked[t], **kw).gen_result()
                compute[(t, name)] = timecostmodel(s, bsz_chunked[t], no_comm=True, **kw).gen_result()
            optimizer[(t, name)] = 0.001 * opt_ms * getattr(profile_hardware_args_list[t], "costmodel_coe", 1.0)
    keys = [(type_of_layer[i], form_strategy(strategies[i])) for i in range(len(strategies))]
    stage_full = get_time_cost_all_stages([full[k] for k in keys], partition)
    stage_compute = get_time_cost_all_stages([compute[k] for k in keys], partition)
    assert len(other_time_cost) == len(stage_compute)
    for i in range(len(other_time_cost)):
        stage_compute[i] += other_time_cost[i]
    result = np.sum(stage_compute) + stage_compute[-1] * (max_chunk - 1)
    ramp = min(pp_deg - 1, max_chunk - 1) * stage_compute[0]
    tail = np.sum(stage_compute[1:])
    result = max(result, max(ramp * 1 / 3, tail * 1 / 3) + max(ramp * 2 / 3, tail * 2 / 3)
                 + stage_compute[0] * max(0, max_chunk + 1 - pp_deg))
    exposed = [stage_full[i] - np.sum(stage_compute[:i + 1]) for i in range(pp_deg)]
    result += max(np.max(exposed), 0)
    # the optimizer step runs once per training step on every stage at the same time: the slowest stage counts
    result += float(np.max(get_time_cost_all_stages([optimizer[k] for k in keys], partition)))
    if return_stage_cost:
        return stage_full, result
    return result
