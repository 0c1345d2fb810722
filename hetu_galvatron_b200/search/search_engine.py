"""The strategy search engine: profiles + hardware tables -> the fastest per-layer plan under a memory budget.

Public surface and file formats follow the reference's ``GalvatronSearchEngine``
(galvatron/core/search_engine/search_engine.py): ``set_search_engine_info`` (:45-50),
``initialize_search_engine`` (:101-106), ``parallelism_optimization`` (:339-537), ``save_results`` (:640-688),
``check_cost_model`` (:691-780), strategy generation (:783-914) and pipeline division (:972-1088).
The search itself is a grid over (batch size, chunks, min/max tensor-parallel degree, vocab sequence
parallelism, embedding ZeRO-3, sp search mode); each grid point runs the dynamic program of
``dynamic_programming.DpOnModel`` over the C++ core.
"""
from __future__ import annotations

import copy
import os
from itertools import product

import numpy as np

from ..utils.config_utils import (array2str, num2str, read_allreduce_bandwidth_config, read_json_config,
                                  read_p2p_bandwidth_config, remap_config, strategy2config, write_json_config)
from ..utils.strategy_utils import form_strategy, print_strategies
from .cost_model import MemoryCostModel, TimeCostModel
from .cost_model_args import ModelArgs, ParallelArgs, ProfileHardwareArgs, ProfileModelArgs, TrainArgs
from .dynamic_programming import DpOnModel
from .log_utils import ensure_log_dir, get_thread_logger

HARDWARE_DIR_DEFAULT = "../../profile_hardware/hardware_configs/"


def _int_keys(d):
    """JSON object keys that are digit strings become ints (recursively)."""
    if not isinstance(d, dict):
        return d
    return {(int(k) if isinstance(k, str) and k.isdigit() else k): _int_keys(v) for k, v in d.items()}


def _powers_of_two(limit: int):
    out, i = [], 1
    while i <= limit:
        out.append(i)
        i *= 2
    return out


def _fit_line(xs, ys):
    """Least-squares line through the profiled points; returns (slope, intercept)."""
    from scipy.optimize import curve_fit

    popt, _ = curve_fit(lambda x, m, c: m * x + c, xs, ys)
    return popt


def _fit_parabola(xs, ys):
    """Least-squares parabola a x^2 + b x + c; returns (a, b, c)."""
    from scipy.optimize import curve_fit

    popt, _ = curve_fit(lambda x, a, b, c: a * x * x + b * x + c, xs, ys)
    return popt


# ========================== pipeline division & chunk helpers ==========================
def pp_division_even(layernum_list, pp_deg):
    total = int(np.sum(layernum_list))
    avg = total // pp_deg
    return [avg] * (pp_deg - 1) + [total - avg * (pp_deg - 1)]


def optimal_chunk_func_default(local_bsz, strategy, microbatch_size, min_tp):
    assert strategy[1] % min_tp == 0
    local_bsz = local_bsz // (strategy[1] // min_tp)
    chunk = np.ceil(local_bsz / microbatch_size)
    return 1 if chunk == 0 else chunk


def check_optimal_chunks(world_size, strategies, optimal_chunk_func, bsz, mbsz_dict, min_tp):
    return {pp: optimal_chunk_func(bsz / (world_size // pp // min_tp), [pp, min_tp, world_size // pp, {"fsdp": 0, "cpt": 0}],
                                   mbsz_dict[pp], min_tp)
            for pp in sorted(set(s[0] for s in strategies))}


def get_layer_costs(layernum_list, layer_costs):
    out = []
    for n, c in zip(layernum_list, layer_costs):
        out += [c] * n
    return out


def get_cost_all_stages(layer_memcosts, pp_stage_division):
    """Sum per stage; one (two) extra leading/trailing entries are the embedding (and head) costs."""
    div = list(copy.deepcopy(pp_stage_division))
    extra = len(layer_memcosts) - int(np.sum(div))
    if extra >= 1:
        div[0] += 1
    if extra == 2:
        div[-1] += 1
    assert int(np.sum(div)) == len(layer_memcosts)
    bounds = np.concatenate([[0], np.cumsum(div)]).astype(int)
    return [np.sum(layer_memcosts[bounds[i]:bounds[i + 1]]) for i in range(len(div))]


def pp_division_memory_balanced(model_args_list, train_args_list, parallel_args_list, profile_model_args_list, layer_num,
                                pp_deg, bsz, mbsz, strategies):
    """Greedy layer -> stage assignment that evens out memory (layers + embedding/head) across stages, used when
    the model has several layer types (reference search_engine.py:972-1047)."""
    n_types = len(layer_num)
    model_args_list = [copy.deepcopy(model_args_list[i]) for i in range(n_types)]
    train_args_list = [copy.deepcopy(train_args_list[i]) for i in range(n_types)]
    parallel_args_list = [copy.deepcopy(parallel_args_list[i]) for i in range(n_types)]
    profile_model_args_list = [copy.deepcopy(profile_model_args_list[i]) for i in range(n_types)]
    for pa in parallel_args_list:
        pa.pipeline_type = "gpipe"
    if pp_deg == 1:
        return [int(np.sum(layer_num))], None
    strategies = [s for s in strategies if s[0] == pp_deg]
    if not strategies:
        return None, None
    gpu_num = strategies[0][0] * strategies[0][1] * strategies[0][2]
    kw = lambda i: dict(model_args=model_args_list[i], train_args=train_args_list[i], parallel_args=parallel_args_list[i],
                        profile_model_args=profile_model_args_list[i])
    per_type = [np.min(MemoryCostModel([pp_deg, 1, gpu_num // pp_deg, {}], global_batch_size=bsz, mbsz=mbsz, min_tp=1, max_tp=1,
                                       **kw(i)).get_memory_cost()["enc_total"]) for i in range(n_types)]
    other = MemoryCostModel(strategies[0], global_batch_size=bsz, mbsz=mbsz, min_tp=1, max_tp=1, **kw(0)).get_memory_cost()["other"][1]
    per_layer = get_layer_costs(layer_num, per_type)
    avg = (np.sum(per_layer) + np.sum(other)) / pp_deg
    divide = [0] * pp_deg
    stage_mem = list(other)
    idx = 0
    for st in range(pp_deg):
        while idx < len(per_layer):
            if st < pp_deg - 1 and avg - stage_mem[st] < 0.5 * per_layer[idx]:
                break
            stage_mem[st] += per_layer[idx]
            idx += 1
            divide[st] += 1
    for st in range(pp_deg - 1):           # no stage above 1.3x the average
        left, right = int(np.sum(divide[:st])), int(np.sum(divide[:st + 1]))
        cur = np.sum(per_layer[left:right]) + other[st]
        while cur > avg * 1.3:
            divide[st] -= 1
            divide[st + 1] += 1
            right -= 1
            cur -= per_layer[right]
    for st in range(pp_deg - 1):           # no empty stage, front to back then back to front
        while divide[st] <= 0:
            divide[st] += 1
            divide[st + 1] -= 1
    for st in range(pp_deg - 1, 0, -1):
        while divide[st] <= 0:
            divide[st] += 1
            divide[st - 1] -= 1
    adjusted = list(other)
    for st in range(pp_deg):
        left, right = int(np.sum(divide[:st])), int(np.sum(divide[:st + 1]))
        adjusted[st] += np.sum(per_layer[left:right])
    return divide, adjusted


def get_pp_stage_for_bsz(strategies, model_args_list, train_args_list, parallel_args_list, profile_model_args_list,
                         layer_num_list, bsz, mbsz_dict, single_layer_even=True):
    out = {}
    for pp_deg in sorted(set(s[0] for s in strategies)):
        if single_layer_even and len(layer_num_list) == 1:
            out[pp_deg] = pp_division_even(layer_num_list, pp_deg)
        else:
            out[pp_deg], _ = pp_division_memory_balanced(model_args_list, train_args_list, parallel_args_list,
                                                         profile_model_args_list, layer_num_list, pp_deg, bsz,
                                                         mbsz_dict[pp_deg], strategies)
    return out


# ========================== the engine ==========================
class GalvatronSearchEngine:
    def __init__(self, args):
        self.args = args
        args.gpu_num = args.num_nodes * args.num_gpus_per_node
        self.layernum_arg_names = None
        self.mem_path = self.time_path = self.model_name = None
        self.time_config = self.memory_config = None
        self.param_sizes = self.act_sizes = None
        self.other_memory_pp_off = self.other_memory_pp_on = None
        self.time_profiled_list = None
        self.use_pipeline_costmodel = args.use_pipeline_costmodel
        self.model_type = "gpt"
        self.optimal_chunk_func = optimal_chunk_func_default
        self.memory_constraint = args.memory_constraint * 1024
        if not hasattr(args, "global_memory_buffer"):
            args.global_memory_buffer = True
        if not hasattr(args, "async_grad_reduce"):
            args.async_grad_reduce = True

    # ---------------- basic information ----------------
    def set_search_engine_info(self, path, model_layer_configs, model_name):
        self.set_model_layer_configs(model_layer_configs)
        self.set_path(path)
        self.set_model_name(model_name)
        self.memory_profiling_path()
        self.time_profiling_path()

    def set_path(self, path):
        self.path = path

    def set_model_type(self, model_type):
        self.model_type = model_type

    def set_model_name(self, name):
        self.model_name = name

    def _profile_path(self, kind: str, override):
        assert self.model_name is not None, "Should specify the model name!"
        name = "%s_profiling_%s_%s.json" % (kind, self.args.mixed_precision, self.model_name)
        folder = override if override is not None else os.path.join(self.path, "configs")
        return os.path.join(folder, name)

    def memory_profiling_path(self):
        if self.mem_path is None:
            self.mem_path = self._profile_path("memory", self.args.memory_profiling_path)
        return self.mem_path

    def time_profiling_path(self):
        if self.time_path is None:
            self.time_path = self._profile_path("computation", self.args.time_profiling_path)
        return self.time_path

    def set_microbatch_func(self, microbatch_size, max_chunk):
        self.optimal_chunk_func = lambda local_bsz, strategy: optimal_chunk_func_default(local_bsz, strategy, microbatch_size)

    def set_model_layer_configs(self, model_layer_configs):
        if model_layer_configs is None:
            return
        self.hiddensize_list = [c["hidden_size"] for c in model_layer_configs]
        self.layernum_list = [c["layer_num"] for c in model_layer_configs]
        self.seqlen_list = [c["seq_len"] for c in model_layer_configs]
        self.num_layertype = len(self.layernum_list)

    # ---------------- initialisation ----------------
    def initialize_search_engine(self, show: bool = True):
        self.generate_strategies()
        self.get_profiled_model_configs()
        self.get_profiled_hardware_configs()
        self.set_cost_models()
        if show:
            self.show_search_info()

    def convert_keys_to_int(self, d):
        return _int_keys(d)

    def _time_profiles(self):
        """Per-layer-type forward time (ms per layer per sample, or a (slope, intercept) fit) and the same for
        the embedding/head part, according to --time_profile_mode."""
        mode = self.args.time_profile_mode
        tc = self.time_config
        layers, other = [], []
        if mode == "static":
            for i in range(self.num_layertype):
                for key, t in tc.items():
                    if key.startswith("layertype_%d_" % i):
                        layers.append(t)
                    if key.startswith("layertype_other_"):
                        other.append(t)
            return layers, other
        for i in range(self.num_layertype):
            seq = self.seqlen_list[i]
            for prefix, sink in (("layertype_%d_" % i, layers), ("layertype_other_", other)):
                xs, ys = [], []
                if mode == "batch":
                    for key, t in tc.items():
                        if key.startswith(prefix) and "_seq%d" % seq in key:
                            b = int(key.split("_")[-2][3:])
                            xs.append(b)
                            ys.append(t * b)
                    assert len(xs) >= 8, "Different bsz in computation profile of %s should not be lower than 8." % prefix
                    sink.append(_fit_line(xs, ys))
                else:  # sequence: time of one sample as a function of the sequence length
                    for key, t in tc.items():
                        if key.startswith(prefix) and "_bsz1_" in key:
                            xs.append(int(key.split("seq")[-1]))
                            ys.append(t)
                    if sink is layers:
                        a, b, c = _fit_parabola(xs, ys)
                        sink.append(a * seq * seq + b * seq + c)
                    else:
                        m, c = _fit_line(xs, ys)
                        sink.append(m * seq + c)
        # the reference collects all layer fits first, then all "other" fits
        return layers, other

    def get_profiled_model_configs(self):
        self.time_config = read_json_config(self.time_profiling_path())
        self.memory_config = _int_keys(read_json_config(self.memory_profiling_path()))
        self.time_profiled_list, self.other_time_profiled_list = self._time_profiles()
        mc = self.memory_config
        self.param_sizes = [0] * self.num_layertype
        self.act_sizes = [{} for _ in range(self.num_layertype)]
        if self.args.memory_profile_mode == "sequence":
            assert self.args.sequence_parallel, "Sequence parallel is required for sequence memory profiling."
            assert self.num_layertype == 1, "Only support num(layertype) == 1 for sequence memory profiling."
            maxseqs = []
            for i in range(self.num_layertype):
                table = mc["layertype_%d_sp" % i]
                seqs = [int(s) for s in table]
                hi, lo = max(seqs), min(seqs)
                maxseqs.append(hi)
                self.param_sizes[i] = table[lo]["parameter_size"]
                self.act_sizes[i] = {tp: v / hi * self.seqlen_list[i] for tp, v in table[hi]["tp_activation_per_bsz_dict"].items()}
            self.other_memory_pp_off = mc["other_memory_pp_off_sp"][maxseqs[0]]
            self.other_memory_pp_on = {"first_stage": mc["other_memory_pp_on_first_sp"][maxseqs[0]],
                                       "last_stage": mc["other_memory_pp_on_last_sp"][maxseqs[-1]]}
            for tp in self.other_memory_pp_off["activation"]:
                self.other_memory_pp_off["activation"][tp] = self.other_memory_pp_off["activation"][tp] / maxseqs[0] * self.seqlen_list[0]
                first = self.other_memory_pp_on["first_stage"]["activation"]
                last = self.other_memory_pp_on["last_stage"]["activation"]
                first[tp] = first[tp] / maxseqs[0] * self.seqlen_list[0]
                last[tp] = last[tp] / maxseqs[-1] * self.seqlen_list[-1]
        elif self.args.memory_profile_mode == "static":
            suffix = "_sp" if self.args.sequence_parallel else ""
            for i in range(self.num_layertype):
                entry = mc["layertype_%d%s" % (i, suffix)][self.seqlen_list[i]]
                self.param_sizes[i] = entry["parameter_size"]
                self.act_sizes[i] = entry["tp_activation_per_bsz_dict"].copy()
            seq_info = num2str(self.seqlen_list, "seq")[3:]
            if seq_info.isdigit():
                seq_info = int(seq_info)
            self.other_memory_pp_off = mc["other_memory_pp_off" + suffix][seq_info]
            self.other_memory_pp_on = {"first_stage": mc["other_memory_pp_on_first" + suffix][seq_info],
                                       "last_stage": mc["other_memory_pp_on_last" + suffix][seq_info]}
        return self.time_config, self.memory_config

    def _hardware_file(self, override, name: str) -> str:
        folder = override if override is not None else os.path.join(self.path, HARDWARE_DIR_DEFAULT)
        return os.path.join(folder, name)

    def get_profiled_hardware_configs(self):
        args = self.args
        tag = "%dnodes_%dgpus_per_node.json" % (args.num_nodes, args.num_gpus_per_node)
        if args.num_nodes * args.num_gpus_per_node == 1:
            # one GPU: no group of more than one rank is ever priced, so no bandwidth table is needed (only
            # --check_cost_model / --explain_plan make sense here)
            self.allreduce_bandwidth, self.allreduce_comm_coe, self.p2p_bandwidth, self.p2p_comm_coe = {}, {"1": 0.0}, {}, {}
            self.overlap_coe, self.sp_allreduce, self.sp_all2all = 1.0, {}, {}
            return self.allreduce_bandwidth, self.p2p_bandwidth, self.overlap_coe, self.sp_allreduce, self.sp_all2all
        args.allreduce_bandwidth_config_path = self._hardware_file(args.allreduce_bandwidth_config_path, "allreduce_bandwidth_" + tag)
        self.allreduce_bandwidth, self.allreduce_comm_coe = read_allreduce_bandwidth_config(
            args.allreduce_bandwidth_config_path, gpu_num=args.gpu_num)
        args.p2p_bandwidth_config_path = self._hardware_file(args.p2p_bandwidth_config_path, "p2p_bandwidth_" + tag)
        self.p2p_bandwidth, self.p2p_comm_coe = read_p2p_bandwidth_config(args.p2p_bandwidth_config_path)
        args.overlap_coe_path = self._hardware_file(args.overlap_coe_path, "overlap_coefficient.json")
        self.overlap_coe = read_json_config(args.overlap_coe_path)["overlap_coe"]
        args.sp_time_path = self._hardware_file(args.sp_time_path, "sp_time_" + tag)
        sp_config = read_json_config(args.sp_time_path)
        self.sp_allreduce = remap_config(sp_config, "allreduce")
        self.sp_all2all = remap_config(sp_config, "all2all")
        return self.allreduce_bandwidth, self.p2p_bandwidth, self.overlap_coe, self.sp_allreduce, self.sp_all2all

    def _bct_fct_coe(self) -> float:
        """Backward / forward ratio: flag, else the time profile's measured value, else the reference's constant 2."""
        v = getattr(self.args, "bct_fct_coe", None)
        if v is None and isinstance(getattr(self, "time_config", None), dict):
            v = self.time_config.get("bct_fct_coe")
        return float(v) if v else 2

    def set_cost_models(self):
        a = self.args
        self.model_args_list, self.train_args_list, self.parallel_args_list = [], [], []
        self.profile_model_args_list, self.profile_hardware_args_list = [], []
        for i in range(self.num_layertype):
            self.model_args_list.append(ModelArgs(parameter_size=self.param_sizes[i], seq_length=self.seqlen_list[i],
                                                  hidden_size=self.hiddensize_list[i], layer_num=self.layernum_list[i]))
            self.train_args_list.append(TrainArgs(mixed_precision=a.mixed_precision != "fp32",
                                                  async_grad_reduce=a.async_grad_reduce,
                                                  pytorch_context_mem=int(getattr(a, "context_mem_mb", None) or 1024),
                                                  memory_layout=getattr(a, "memory_layout", "fsdp"),    # the command line defaults to "engine"
                                                  grad_bytes=2 if getattr(a, "grad_dtype", "fp32") == "bf16" else 4,
                                                  fused_engine=getattr(a, "comm_impl", "nccl") == "fused"))
            self.parallel_args_list.append(ParallelArgs(use_zero2_for_dp=a.default_dp_type == "zero2", disable_vtp=a.disable_vtp,
                                                        sequence_parallel=a.sequence_parallel, sp_space=a.sp_space,
                                                        pipeline_type=a.pipeline_type, optimal_chunk_func=self.optimal_chunk_func,
                                                        cp_size=getattr(self, "cp_size", 1)))
            self.profile_model_args_list.append(ProfileModelArgs(
                tp_activation_per_bsz_dict=self.act_sizes[i], other_memory_pp_off=self.other_memory_pp_off,
                other_memory_pp_on=self.other_memory_pp_on, forward_computation_time=self.time_profiled_list[i],
                other_time_profiled=self.other_time_profiled_list[0],
                optimizer_time=float((self.time_config or {}).get("optimizer_ms_layertype_%d" % i, 0.0))))
            self.profile_hardware_args_list.append(ProfileHardwareArgs(
                bct_fct_coe=self._bct_fct_coe(), extra_overhead=0, comm_coe_dict=self.allreduce_comm_coe, dp_overlap_coe=self.overlap_coe,
                bct_overlap_coe=self.overlap_coe, p2p_comm_coe_dict=self.p2p_comm_coe, costmodel_coe=a.costmodel_coe,
                allreduce_dict=self.sp_allreduce, all2all_dict=self.sp_all2all,
                fused_comm_exposed=getattr(a, "fused_comm_exposed", 1.0)))

    # ---------------- the search ----------------
    def _search_grid(self):
        """Axes of the outer grid (reference search_engine.py:349-376)."""
        a = self.args
        min_tps = [t for t in _powers_of_two(a.gpu_num) if t <= a.max_tp_deg]
        if a.disable_vtp:
            min_tps = [1]
        if not a.global_memory_buffer:
            max_tps, sp_modes = [a.max_tp_deg], [1, 3]
        else:
            max_tps, sp_modes = min_tps, [1, 2, 3]          # 1: tp, 2: sp, 3: tp+sp
        if a.sp_space == "tp+sp":
            vsps = [0, 1]
        elif a.sp_space == "tp":
            vsps, sp_modes = [0], [1]
        else:
            raise AssertionError("Only sp mode unsupport now.")
        embed_sdps = [0] if a.disable_sdp else [0, 1]
        return min_tps, max_tps, vsps, embed_sdps, sp_modes

    def _search_for_chunk(self, bsz, chunk, min_tp, max_tp, vsp, embed_sdp, sp_modes, all_strategies):
        a = self.args
        log_dir = ensure_log_dir(a.log_dir + "/%s_%dnodes_%dgpus_%dGB" % (self.model_name, a.num_nodes, a.num_gpus_per_node,
                                                                        self.memory_constraint // 1024))
        logger = get_thread_logger(bsz, chunk, min_tp, max_tp, vsp, embed_sdp, log_dir)
        logger.info(f"Starting search for bsz={bsz}, chunk={chunk}, min_tp={min_tp}, max_tp={max_tp}, vsp={vsp}, embed_sdp={embed_sdp}")
        results = {}
        for sp_search in sp_modes:
            if (sp_search == 1 and vsp == 1) or (sp_search == 2 and vsp == 0):
                continue
            cand = [s for s in all_strategies if min_tp <= s[1] <= max_tp]
            cand = [s for s in cand if chunk <= bsz // (a.gpu_num // s[0] // min_tp)]
            if sp_search == 1:
                cand = [s for s in cand if not s[-1].get("sp", 0)]
            if sp_search == 2:
                cand = [s for s in cand if "sp" not in s[-1] or s[-1]["sp"] == 1]
            if not cand:
                continue
            pps = sorted(set(s[0] for s in cand))
            pps = [pp for pp in pps if pp * min_tp <= a.gpu_num and bsz % (a.gpu_num // pp // min_tp) == 0]
            if not pps:
                continue
            cand = [s for s in cand if s[0] in pps]
            # micro-batch size per pipeline degree at tp = min_tp; keep only strategies whose real chunk count
            # equals the searched one
            mbsz_dict = {pp: (bsz // (a.gpu_num // pp // min_tp) + chunk - 1) // chunk for pp in pps}
            cand = [s for s in cand
                    if chunk == (bsz // (a.gpu_num // s[0] // min_tp) + mbsz_dict[s[0]] - 1) // mbsz_dict[s[0]]]
            if not cand:
                continue
            pp_stage_dict = get_pp_stage_for_bsz(cand, self.model_args_list, self.train_args_list, self.parallel_args_list,
                                                 self.profile_model_args_list, self.layernum_list, bsz, mbsz_dict)
            results[sp_search] = self.dynamic_programming(cand, bsz, chunk, mbsz_dict, pp_stage_dict, min_tp, max_tp, vsp,
                                                          embed_sdp, sp_search, logger)
            results[sp_search]["pp_stage_dict"] = copy.deepcopy(pp_stage_dict)
        return results

    def parallelism_optimization(self):
        print("=" * 25, "Galvatron Search Engine Start Searching", "=" * 25)
        self.set_searching_bsz()
        print("-----", "[Searching Memory Info]", "Memory constraint:", self.memory_constraint, "MB", "-----")
        a = self.args
        self.search_history = {}
        all_strategies = copy.deepcopy(self.strategies)
        min_tps, max_tps, vsps, embed_sdps, sp_modes = self._search_grid()
        tasks = []
        for bsz in self.BSZs:
            chunks = [a.settle_chunk] if a.settle_chunk != -1 else range(1, bsz + 1)
            for chunk in chunks:
                if bsz % chunk != 0:
                    continue
                for min_tp, max_tp, vsp, embed_sdp in product(min_tps, max_tps, vsps, embed_sdps):
                    if min_tp <= max_tp:
                        tasks.append((bsz, chunk, min_tp, max_tp, vsp, embed_sdp))
        results = {}

        def run(task):
            return task, self._search_for_chunk(*task, sp_modes, all_strategies)

        if a.parallel_search and len(tasks) > 1:
            import concurrent.futures
            import multiprocessing

            workers = a.worker if getattr(a, "worker", 0) > 0 else multiprocessing.cpu_count() * 2
            workers = min(workers, len(tasks))
            print(f"Starting parallel search with {workers} threads for {len(tasks)} tasks...")
            with concurrent.futures.ThreadPoolExecutor(max_workers=workers) as ex:
                for task, res in ex.map(run, tasks):
                    results[task] = res
        else:
            for task in tasks:
                print("Start processing: bsz=%d, chunk=%d, min_tp=%d, max_tp=%d, vsp=%d, embed_sdp=%d" % task, flush=True)
                results[task] = run(task)[1]

        best, best_key = None, None
        max_throughput = -1
        for task in tasks:                       # first strictly better result wins, in grid order
            for sp_search, res in results[task].items():
                if res["throughput"] > max_throughput:
                    max_throughput, best, best_key = res["throughput"], res, task
        if max_throughput > 0:
            bsz, chunk, min_tp, max_tp, vsp, embed_sdp = best_key
            print("\nFinal results of max memory %d MB:" % self.memory_constraint)
            best["vsp"], best["embed_sdp"] = vsp, embed_sdp
            print(f"Optimal bsz = {bsz} Optimal chunk = {chunk} Optimal vocab tp = {best['vtp']} Optimal vocab sp = {vsp} "
                  f"Optimal embed sdp = {embed_sdp} Max throughput={best['throughput']} samples/s")
            print(f"pp_deg={best['min_pp_deg']} Minimized timecost={best['min_cost']} Memory remaining={best['mem_remain']} "
                  f"Memory cost={best['mem_cost']}")
            print(f"Min_tp={min_tp} Max_tp={max_tp} ")
            print_strategies(best["min_res_list"])
            self.best_result = best
            self.save_results(best, bsz, chunk, best["pp_stage_dict"])
        else:
            print("No valid configuration found.")
        print("-----------------------------------------")
        print("=" * 25, "Galvatron Search Engine End Searching", "=" * 25)
        return max_throughput

    def set_searching_bsz(self):
        a = self.args
        if a.settle_bsz is not None and a.settle_bsz > 0:
            self.min_bsz = self.max_bsz = a.settle_bsz
            self.bsz_scale = 0
            self.BSZs = [a.settle_bsz]
            print("-----", "[Searching Batch Sizes Info]", "Settle bsz:", a.settle_bsz, "-----")
            return
        self.bsz_scale = a.bsz_scale
        if a.recommend_min_bsz:
            rec = self.recommend_min_bsz(self.bsz_scale)
            a.min_bsz = rec if rec > 0 else a.min_bsz
        self.min_bsz = max(a.min_bsz, self.bsz_scale) // self.bsz_scale * self.bsz_scale
        if a.max_bsz % self.bsz_scale:
            self.max_bsz = int(np.ceil(a.max_bsz / self.bsz_scale) * self.bsz_scale)
        else:
            self.max_bsz = a.max_bsz + self.bsz_scale
        self.BSZs = list(range(self.min_bsz, self.max_bsz, self.bsz_scale))
        self.max_bsz = self.BSZs[-1]
        print("-----", "[Searching Batch Sizes Info]", "Min bsz:", self.min_bsz, "Max bsz:", self.max_bsz, "bsz_scale:",
              self.bsz_scale, "-----")

    def recommend_min_bsz(self, scale):
        """Start the batch-size sweep 65 % of the way between the largest batches pure DP / SDP / TP can hold."""
        a = self.args
        if a.search_space not in ("full", "dp+pp", "dp+tp"):
            return -1
        baselines = []
        if not a.disable_dp:
            baselines.append([1, 1, a.gpu_num, {"fsdp": 0}])
        if not a.disable_sdp:
            baselines.append([1, 1, a.gpu_num, {"fsdp": 1}])
        if not a.disable_tp:
            baselines.append([1, a.gpu_num, 1, {"fsdp": 0}])
        limits = [self.estimate_strategy_max_bsz([s], scale) for s in baselines]
        hi, lo = np.max(limits), np.min(limits)
        start = int((lo * 0.35 + hi * 0.65) // scale * scale)
        return start if start > scale else scale

    def _dp_on_model(self, strategies, pp_stage_dict, logger=None, full=True):
        a = self.args
        extra = dict(search_history=self.search_history, model_microbatch_after_dp=a.use_pipeline_costmodel,
                     pipeline_type=a.pipeline_type, logger=logger) if full else {}
        return DpOnModel(strategies, MemoryCostModel, TimeCostModel, model_args_list=self.model_args_list,
                         train_args_list=self.train_args_list, parallel_args_list=self.parallel_args_list,
                         profile_model_args_list=self.profile_model_args_list,
                         profile_hardware_args_list=self.profile_hardware_args_list, max_mem=self.memory_constraint,
                         layer_num=self.layernum_list, sequence_len=self.seqlen_list, multi_layer_type=True,
                         pp_stage_dict=pp_stage_dict, comm_coe_dict=self.allreduce_comm_coe, gpu_num=a.gpu_num, config=a,
                         **extra)

    def estimate_strategy_max_bsz(self, strategies, scale):
        bsz = scale
        while True:
            pp_stage_dict = get_pp_stage_for_bsz(strategies, self.model_args_list, self.train_args_list, self.parallel_args_list,
                                                 self.profile_model_args_list, self.layernum_list, bsz, {1: bsz})
            model = self._dp_on_model(strategies, pp_stage_dict, full=False)
            _, _, pp, _, _, _ = model.fit(bsz, 1, 1, 0, 1, 1, print_=False, mbsz_dict={1: bsz})
            if pp == -1:
                return bsz - scale
            bsz += scale

    def dynamic_programming(self, strategies, bsz, chunk, mbsz_dict, pp_stage_dict, min_tp, max_tp, vsp, embed_sdp, sp_search,
                            logger):
        a = self.args
        logger.info(f"bsz={bsz} {pp_stage_dict}")
        model = self._dp_on_model(strategies, pp_stage_dict, logger=logger)
        logger.info(f"****Searching with bsz={bsz} chunk={chunk} min_tp={min_tp} max_tp={max_tp} vsp={vsp} "
                    f"embed_sdp={embed_sdp} sp_search={sp_search}****")
        logger.info(f"Chunk_dict for bsz {bsz}: {check_optimal_chunks(a.gpu_num, strategies, self.optimal_chunk_func, bsz, mbsz_dict, min_tp)}")
        logger.info(f"Mbsz_dict for bsz {bsz}: {mbsz_dict}")
        cost, plan, pp, remain, mem, vtp = model.fit(bsz, min_tp, max_tp, vsp, embed_sdp, sp_search, mbsz_dict=mbsz_dict)
        throughput = bsz / cost
        logger.info(f"[Optimal pp_deg={pp}] Minimized timecost={cost} Memory remaining={remain} Memory cost={mem} Vocab tp={vtp}")
        logger.info(f"Max throughput={throughput} samples/s")
        print_strategies(plan, logger)
        return {"min_cost": cost, "min_res_list": plan, "min_pp_deg": pp, "mem_remain": remain, "mem_cost": mem,
                "throughput": throughput, "vtp": vtp}

    # ---------------- output ----------------
    def result_config(self, re, bsz, chunk, pp_stage_dict) -> dict:
        """The plan JSON of a search result (keys of the reference's save_results, search_engine.py:651-668)."""
        plan = re["min_res_list"]
        if isinstance(plan, list) and isinstance(plan[0], list) and isinstance(plan[0][0], list):
            plan = [s for stage in plan for s in stage]
        config = strategy2config(plan)
        config["checkpoint"] = array2str([1 if s[-1].get("cpt") else 0 for s in plan])
        config["global_bsz"] = bsz
        config["chunks"] = chunk
        config["pp_division"] = array2str(pp_stage_dict[config["pp_deg"]])
        config["pipeline_type"] = self.args.pipeline_type
        config["default_dp_type"] = self.args.default_dp_type
        config["vtp"], config["vsp"], config["embed_sdp"] = re["vtp"], re["vsp"], re["embed_sdp"]
        if getattr(self.args, "sequence_parallel", False):
            config["sequence_parallel"] = 1      # the runtime reads it; the reference passes --sequence-parallel by hand
        return config

    def output_config_name(self) -> str:
        a = self.args
        off = [n for n, flag in (("dp", a.disable_dp), ("tp", a.disable_tp), ("pp", a.disable_pp), ("sdp", a.disable_sdp),
                                 ("ckpt", a.disable_ckpt), ("tpconsec", a.disable_tp_consec)) if flag]
        name = "galvatron_config_%s_%dnodes_%dgpus_per_node_%dGB" % (self.model_name, a.num_nodes, a.num_gpus_per_node,
                                                                    self.memory_constraint // 1024)
        name += "_%s" % a.mixed_precision
        name += "_bsz%d" % a.settle_bsz if a.settle_bsz > 0 else ""
        name += "_[%s_off]" % "_".join(off) if off else ""
        return name + ".json"

    def save_results(self, results, bsz, chunk, pp_stage_dict):
        re = results
        if not (re["min_pp_deg"] > 0 and re["min_res_list"] is not None):
            return None
        config = self.result_config(re, bsz, chunk, pp_stage_dict)
        folder = self.args.output_config_path
        if folder is None:
            folder = os.path.join(self.path, "configs/")
        path = os.path.join(folder, self.output_config_name())
        print(path)
        write_json_config(config, path)
        print("Already written optimized parallelism config into galvatron config file %s!" % path)
        self.output_path = path
        return path

    def check_cost_model(self, bsz, chunk, min_tp):
        """Developer aid: print, for every strategy, the predicted per-stage memory and the pipeline time, so they
        can be compared with measured numbers (reference search_engine.py:691-780). Returns the table."""
        from .cost_model import pipeline_costmodel

        a = self.args
        strategies = [s for s in copy.deepcopy(self.strategies) if s[1] >= min_tp]
        pps = sorted(set(s[0] for s in strategies))
        pps = [pp for pp in pps if pp * min_tp <= a.gpu_num and bsz % (a.gpu_num // pp // min_tp) == 0]
        strategies = [s for s in strategies if s[0] in pps]
        mbsz_dict = {pp: (bsz // (a.gpu_num // pp // min_tp) + chunk - 1) // chunk for pp in pps}
        pp_stage_dict = get_pp_stage_for_bsz(strategies, self.model_args_list, self.train_args_list, self.parallel_args_list,
                                             self.profile_model_args_list, self.layernum_list, bsz, mbsz_dict)
        table = []
        for s in strategies:
            pp = s[0]
            stage_mem = []
            for stage_idx in range(pp):
                per_type = []
                other = None
                for i in range(self.num_layertype):
                    pa = copy.deepcopy(self.parallel_args_list[i])
                    pa.chunks = chunk
                    m = MemoryCostModel(s, global_batch_size=bsz, mbsz=mbsz_dict[pp], min_tp=min_tp, max_tp=a.max_tp_deg,
                                        stage_idx=stage_idx, model_args=self.model_args_list[i], train_args=self.train_args_list[i],
                                        parallel_args=pa, profile_model_args=self.profile_model_args_list[i]).get_memory_cost()
                    per_type.append(m["enc_total"])
                    other = other or m["other"]
                layers = get_layer_costs(self.layernum_list, per_type)
                div = pp_stage_dict[pp]
                lo, hi = int(np.sum(div[:stage_idx])), int(np.sum(div[:stage_idx + 1]))
                vtp = min(other) if other else None
                stage_mem.append(float(np.sum(layers[lo:hi]) + (other[vtp][stage_idx] if other else 0)))
            other_time = [0.0] * pp
            t = pipeline_costmodel(TimeCostModel, self.layernum_list, self.model_args_list, self.train_args_list,
                                   self.parallel_args_list, self.profile_model_args_list, self.profile_hardware_args_list,
                                   [s] * int(np.sum(self.layernum_list)), pp_stage_dict[pp], chunk, bsz, min_tp, other_time)
            table.append({"strategy": form_strategy(s), "stage_memory_mb": stage_mem, "time_s": float(t)})
            print(form_strategy(s), "memory per stage (MB):", ["%.0f" % m for m in stage_mem], "time (s): %.4f" % t)
        return table

    def explain_plan(self, plan: dict):
        """Price an existing strategy JSON (a dict in the plan-file format) with the engine's cost models: per-stage
        memory (layers + embedding / head at the plan's vocab-tp degree), per-stage time and the pipelined step time.
        Returns ``{"stage_memory_mb", "stage_time_s", "step_time_s", "throughput_samples_per_s", "strategies"}``."""
        from ..utils.config_utils import config2strategy, str2array
        from .cost_model import pipeline_costmodel

        a = self.args
        pp, tps, cps, consec, dpt, use_sp, vtp, vsp, _ = config2strategy(plan)
        ckpt = str2array(plan["checkpoint"]) if "checkpoint" in plan else [0] * len(tps)
        bsz, chunk = plan["global_bsz"], plan["chunks"]
        division = str2array(plan["pp_division"]) if "pp_division" in plan else pp_division_even(self.layernum_list, pp)
        stage_gpus = a.gpu_num // pp
        strategies = []
        for i, tp in enumerate(tps):
            info = {"fsdp": int(dpt[i])}
            dp = stage_gpus // tp // cps[i]
            if tp > 1 and dp > 1:
                info["tp"] = int(consec[i])
            if ckpt[i]:
                info["cpt"] = 1
            if use_sp[i]:
                info["sp"] = 1
            strategies.append([pp, tp, dp, info])
        min_tp = min(min(tps), vtp)
        mbsz = (bsz // (a.gpu_num // pp // min_tp) + chunk - 1) // chunk
        type_of_layer = [t for t, n in enumerate(self.layernum_list) for _ in range(n)]
        stage_of_layer = [st for st, n in enumerate(division) for _ in range(n)]
        stage_mem = [0.0] * pp
        other = None
        for i, s in enumerate(strategies):
            t = type_of_layer[i]
            pa = copy.deepcopy(self.parallel_args_list[t])
            pa.chunks = chunk
            pa.pipeline_type = plan.get("pipeline_type", a.pipeline_type)
            pa.use_zero2_for_dp = plan.get("default_dp_type", a.default_dp_type) == "zero2"
            m = MemoryCostModel(s, global_batch_size=bsz, mbsz=mbsz, min_tp=min_tp, max_tp=a.max_tp_deg, stage_idx=stage_of_layer[i],
                                vsp=vsp, embed_sdp=bool(plan.get("embed_sdp", 0)), model_args=self.model_args_list[t],
                                train_args=self.train_args_list[t], parallel_args=pa,
                                profile_model_args=self.profile_model_args_list[t]).get_memory_cost()
            stage_mem[stage_of_layer[i]] += float(m["enc_total"])
            if other is None and vtp in m["other"]:
                other = m["other"][vtp]
        if other is not None:
            stage_mem = [x + float(o) for x, o in zip(stage_mem, other)]
        stage_time, step = pipeline_costmodel(TimeCostModel, self.layernum_list, self.model_args_list, self.train_args_list,
                                              self.parallel_args_list, self.profile_model_args_list,
                                              self.profile_hardware_args_list, strategies, division, chunk, bsz, min_tp,
                                              [0.0] * pp, return_stage_cost=True)
        return {"stage_memory_mb": stage_mem, "stage_time_s": [float(x) for x in stage_time], "step_time_s": float(step),
                "throughput_samples_per_s": bsz / float(step), "strategies": [form_strategy(s) for s in strategies]}

    # ---------------- strategy space ----------------
    def generate_strategies(self):
        a = self.args
        strategies = self.generate_dp_tp_pp_sdp()
        if a.search_space == "dp+tp":
            a.disable_sdp, a.disable_pp = 1, 1
        elif a.search_space == "dp+pp":
            a.disable_sdp, a.disable_tp = 1, 1
        elif a.search_space == "3d":
            a.disable_sdp = 1
        if a.search_space in ("3d", "dp", "tp", "pp", "sdp"):
            self.strategies = strategies
            a.disable_ckpt = 1
            return strategies
        assert not (a.disable_sdp and a.disable_dp)

        def allowed(s):
            info = s[-1]
            if s[2] > 1 and "fsdp" in info:
                if a.disable_dp and info["fsdp"] == 0:
                    return False
                if a.disable_sdp and info["fsdp"] == 1:
                    return False
            if a.disable_tp and s[1] > 1:
                return False
            if a.disable_pp and s[0] > 1:
                return False
            if a.disable_tp_consec and "tp" in info and info["tp"] == 0:
                return False
            return s[1] <= a.max_tp_deg and s[0] <= a.max_pp_deg

        strategies = [s for s in strategies if allowed(s)]
        if not a.disable_ckpt:
            with_ckpt = copy.deepcopy(strategies)
            for s in with_ckpt:
                s[-1]["cpt"] = 1
            strategies = strategies + with_ckpt
        self.strategies = strategies
        return strategies

    def generate_dp_tp_pp_sdp(self, gpu_num=None, search_space=None):
        a = self.args
        gpu_num = a.gpu_num if gpu_num is None else gpu_num
        space = a.search_space
        degrees = _powers_of_two(gpu_num)

        def variants(pp, tp, with_sdp):
            dp = gpu_num // (pp * tp)
            fs = (0, 1) if with_sdp else (0,)
            if tp == 1 or tp == gpu_num / pp:
                return [[pp, tp, dp, {}]] if dp == 1 else [[pp, tp, dp, {"fsdp": f}] for f in fs]
            return [[pp, tp, dp, {"tp": c, "fsdp": f}] for c in (0, 1) for f in fs]

        if space == "full":
            strategies = [s for pp in degrees for tp in degrees if pp * tp <= gpu_num for s in variants(pp, tp, True)]
        elif space == "dp+tp":
            strategies = [s for tp in degrees for s in variants(1, tp, False)]
        elif space == "dp+pp":
            strategies = [s for pp in degrees for s in variants(pp, 1, False)]
        elif space == "3d":
            strategies = [[2, 2, gpu_num // 4, {"tp": 1, "fsdp": 0}]]
        elif space == "dp":
            strategies = [[1, 1, gpu_num, {"fsdp": 0}]]
        elif space == "sdp":
            strategies = [[1, 1, gpu_num, {"fsdp": 1}]]
        elif space == "tp":
            strategies = [[1, a.max_tp_deg, gpu_num // a.max_tp_deg, {"fsdp": 0}]]
            if strategies[0][2] > 1:
                strategies[0][-1]["tp"] = 1
        elif space == "pp":
            strategies = [[a.max_pp_deg, 1, gpu_num // a.max_pp_deg, {"fsdp": 0}]]
        else:
            raise ValueError("unknown search space %r" % space)
        # sequence-parallel flavour of every tensor-parallel strategy
        if a.sp_space in ("tp", "sp"):
            for s in strategies:
                if s[1] > 1:
                    s[-1]["sp"] = 0 if a.sp_space == "tp" else 1
            return strategies
        out = []
        for s in strategies:
            if s[1] > 1:
                for flag in (0, 1):
                    c = copy.deepcopy(s)
                    c[-1]["sp"] = flag
                    out.append(c)
            else:
                out.append(copy.deepcopy(s))
        return out

    def show_search_info(self):
        bar = "=" * 80
        a = self.args
        print(bar)
        print("--- Optimization Configs ----")
        print("Memory constraint: %d GB" % a.memory_constraint)
        print("Pipeline Type:", a.pipeline_type)
        print("Default DP Type:", a.default_dp_type)
        print("Mixed Precision:", a.mixed_precision)
        print("Search Space:")
        print_strategies(self.strategies)
        print(bar)
        print("---- Environment Configs ----")
        print("Allreduce Bandwidth (GB/s):", self.allreduce_bandwidth)
        print("Allreduce Communication Coefficient (ms/MB):", self.allreduce_comm_coe)
        print("P2P Bandwidth (GB/s):", self.p2p_bandwidth)
        print("P2P Communication Coefficient (ms/MB):", self.p2p_comm_coe)
        print("Overlap coefficient:", self.overlap_coe)
        print(bar)
        print("------- Model Configs -------")
        print("Model Name:", self.model_name)
        print("Num layertype:", self.num_layertype)
        print("Layer_num:", self.layernum_list)
        print("Hidden_size:", self.hiddensize_list)
        print("Seq_len:", self.seqlen_list)
        print(bar)
        print("--- Model Computation Configs ---")
        print("Forward computation time:", self.time_profiled_list)
        print(bar)
        print("--- Model Memory Configs ---")
        print("Parameter Memory Cost:", self.param_sizes)
        print("Activation Memory Cost of Different TP degree (per bsz):")
        print(self.act_sizes)
        print("Other Memory Cost (pp = 1):")
        print(self.other_memory_pp_off)
        print("Other Memory Cost (pp > 1):")
        print(self.other_memory_pp_on)
        print(bar)
