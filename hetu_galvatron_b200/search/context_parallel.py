"""Context parallelism as an outer dimension of the strategy search.

The reference runs zigzag context parallelism (galvatron/core/runtime/tensor_parallel/transformer.py:2335-2680,
``--global_cp_deg`` / ``cp_sizes_enc``) but never searches it: its strategies have no cp entry and
``strategy2config`` writes none (galvatron/utils/config_utils.py:46-57). Here a uniform degree ``c`` is searched on top
of the unchanged layer-wise search: for every ``c`` the job is seen as ``world / c`` GPUs working on sequences of
length ``s / c`` with

* forward time per layer and sample = profiled time / c (the zigzag split balances the causal attention work)
  + the time to gather K and V from the other ``c - 1`` ranks, which scales with the batch like compute does and whose
  backward (reduce-scatter of dK / dV and the re-gather under recomputation) is covered by the backward / forward ratio;
* activation memory per sample / c, parameters unchanged; context-parallel ranks are data-parallel for the weights,
  so ZeRO shards and the gradient reduction span ``c x dp`` ranks (``ParallelArgs.cp_size``);
* tensor-parallel messages of ``s / c`` tokens.

The best (throughput, c) wins; its plan carries ``cp_sizes_enc = c`` for every layer and ``vcp = c``.
"""
from __future__ import annotations

import copy
import os
from typing import Dict, List, Optional

import numpy as np

from ..utils.config_utils import array2str, read_json_config, write_json_config
from .cost_model import _coe
from .search_engine import GalvatronSearchEngine


def kv_gather_ms_per_sample(seq_len: int, kv_hidden: int, cp: int, comm_coe_dict: dict, elem_bytes: int = 2) -> float:
    """Forward K + V all-gather of one layer for one sample: (c - 1) / c of ``2 x seq x kv_hidden`` elements cross
    the fabric at the bus bandwidth of a group of ``c`` ranks (context-parallel ranks are strided by the tp degree)."""
    if cp <= 1:
        return 0.0
    mb = 2.0 * seq_len * kv_hidden * elem_bytes / 2 ** 20
    coe = None
    for key in ("%d_0" % cp, "%d" % cp, "%d_1" % cp):
        if key in comm_coe_dict:
            coe = comm_coe_dict[key]
            break
    if coe is None:
        coe = _coe(comm_coe_dict, cp)
    return (cp - 1) / cp * mb * coe


def _scale_activation_tables(engine: GalvatronSearchEngine, cp: int) -> None:
    engine.act_sizes = [{k: v / cp for k, v in table.items()} for table in engine.act_sizes]

    def shrink(entry: dict) -> dict:
        out = copy.deepcopy(entry)
        out["activation"] = {k: v / cp for k, v in entry["activation"].items()}
        return out

    engine.other_memory_pp_off = shrink(engine.other_memory_pp_off)
    engine.other_memory_pp_on = {k: shrink(v) for k, v in engine.other_memory_pp_on.items()}


def sub_engine(args, path: str, model_layer_configs: List[dict], model_name: str, cp: int) -> Optional[GalvatronSearchEngine]:
    """The engine that searches ``world / cp`` GPUs with the profiles rescaled for context-parallel degree ``cp``."""
    a = copy.deepcopy(args)
    world = a.num_nodes * a.num_gpus_per_node
    if world % cp or world // cp < 1:
        return None
    probe = GalvatronSearchEngine(copy.deepcopy(args))
    probe.set_search_engine_info(path, model_layer_configs, model_name)
    # the hardware tables are those of the whole machine, whatever the sub-world's size
    tag = "%dnodes_%dgpus_per_node.json" % (a.num_nodes, a.num_gpus_per_node)
    def folder(override, name):
        # an engine that was already initialised has rewritten these flags from folders into file paths
        if override is not None and str(override).endswith(".json"):
            return os.path.dirname(override)
        return os.path.dirname(probe._hardware_file(override, name))

    a.allreduce_bandwidth_config_path = folder(a.allreduce_bandwidth_config_path, "allreduce_bandwidth_" + tag)
    a.p2p_bandwidth_config_path = folder(a.p2p_bandwidth_config_path, "p2p_bandwidth_" + tag)
    a.overlap_coe_path = folder(a.overlap_coe_path, "overlap_coefficient.json")
    a.sp_time_path = folder(a.sp_time_path, "sp_time_" + tag)
    a.memory_profiling_path = os.path.dirname(probe.memory_profiling_path())
    a.time_profiling_path = os.path.dirname(probe.time_profiling_path())
    full = {k: read_json_config(os.path.join(getattr(a, attr), name)) for k, attr, name in (
        ("allreduce", "allreduce_bandwidth_config_path", "allreduce_bandwidth_" + tag),
        ("p2p", "p2p_bandwidth_config_path", "p2p_bandwidth_" + tag), ("sp", "sp_time_path", "sp_time_" + tag))}
    if a.num_gpus_per_node % cp == 0:            # context-parallel groups stay inside a node where they can
        a.num_gpus_per_node //= cp
    else:
        assert cp % a.num_gpus_per_node == 0 and a.num_nodes % (cp // a.num_gpus_per_node) == 0, \
            "context-parallel degree must divide the GPUs of a node, or be a multiple of them that divides the job"
        a.num_nodes //= cp // a.num_gpus_per_node
        a.num_gpus_per_node = 1
    a.max_tp_deg = min(a.max_tp_deg, a.num_nodes * a.num_gpus_per_node)
    a.max_pp_deg = min(a.max_pp_deg, a.num_nodes * a.num_gpus_per_node)
    eng = GalvatronSearchEngine(a)
    eng.set_search_engine_info(path, model_layer_configs, model_name)
    eng.generate_strategies()
    eng.get_profiled_model_configs()
    # read the whole machine's tables under the sub-world's size
    from ..utils.config_utils import read_allreduce_bandwidth_config, read_p2p_bandwidth_config, remap_config

    sub_world = a.num_nodes * a.num_gpus_per_node
    if sub_world >= 2:
        eng.allreduce_bandwidth, eng.allreduce_comm_coe = read_allreduce_bandwidth_config(full["allreduce"], gpu_num=sub_world)
    else:
        eng.allreduce_bandwidth, eng.allreduce_comm_coe = {"1": float("inf")}, {"1": 0}
    eng.p2p_bandwidth, eng.p2p_comm_coe = read_p2p_bandwidth_config(full["p2p"])
    eng.overlap_coe = read_json_config(os.path.join(a.overlap_coe_path, "overlap_coefficient.json"))["overlap_coe"]
    eng.sp_allreduce, eng.sp_all2all = remap_config(full["sp"], "allreduce"), remap_config(full["sp"], "all2all")
    if cp > 1:
        _, whole_coe = read_allreduce_bandwidth_config(full["allreduce"], gpu_num=world)
        # gradient reduction spans cp x dp ranks: keep the whole machine's entries beside the sub-world's
        eng.allreduce_comm_coe = {**whole_coe, **eng.allreduce_comm_coe}
        elem = 4 if a.mixed_precision == "fp32" else 2
        scaled = []
        for i, t in enumerate(eng.time_profiled_list):
            kv_hidden = model_layer_configs[i].get("kv_hidden_size", model_layer_configs[i]["hidden_size"])
            kv = kv_gather_ms_per_sample(model_layer_configs[i]["seq_len"], kv_hidden, cp, whole_coe, elem)
            if isinstance(t, np.ndarray):        # (slope, intercept) of a batch-size fit
                scaled.append(t / cp + np.array([kv, 0.0]))
            else:
                scaled.append(t / cp + kv)
        eng.time_profiled_list = scaled
        eng.other_time_profiled_list = [t / cp for t in eng.other_time_profiled_list]
        _scale_activation_tables(eng, cp)
        eng.seqlen_list = [s // cp for s in eng.seqlen_list]
    eng.cp_size = cp
    eng.set_cost_models()
    return eng


def search_with_context_parallel(args, path: str, model_layer_configs: List[dict], model_name: str,
                                 max_cp_deg: int = 1) -> Dict[str, object]:
    """Run the layer-wise search for cp = 1, 2, 4, ... <= ``max_cp_deg`` and keep the best plan.

    Returns ``{"throughput", "cp", "config", "path", "per_cp": {cp: throughput}}`` (throughput in samples / s; -1 when
    nothing fits)."""
    out_dir = args.output_config_path if getattr(args, "output_config_path", None) else os.path.join(path, "configs")
    best: Dict[str, object] = {"throughput": -1, "cp": 1, "config": None, "path": None, "per_cp": {}}
    cp = 1
    world = args.num_nodes * args.num_gpus_per_node
    while cp <= max_cp_deg and cp <= world:
        eng = sub_engine(args, path, model_layer_configs, model_name, cp) if world % cp == 0 else None
        if eng is not None:
            eng.args.output_config_path = os.path.join(out_dir, "_cp%d" % cp)
            tp = eng.parallelism_optimization()
            best["per_cp"][cp] = tp
            if tp > best["throughput"] and getattr(eng, "output_path", None):
                config = read_json_config(eng.output_path)
                n = len(config["tp_sizes_enc"].split(","))
                config["cp_sizes_enc"] = array2str([cp] * n)
                config["vcp"] = cp
                best.update(throughput=tp, cp=cp, config=config)
        cp *= 2
    if best["config"] is not None:
        full = GalvatronSearchEngine(copy.deepcopy(args))
        full.set_search_engine_info(path, model_layer_configs, model_name)
        best["path"] = os.path.join(out_dir, full.output_config_name())
        write_json_config(best["config"], best["path"])
        print("Context-parallel search: best cp = %d, throughput %.4f samples/s %s -> %s" % (
            best["cp"], best["throughput"], best["per_cp"], best["path"]))
    return best
