"""Search-engine command-line flags. Names and defaults are the reference's (galvatron/core/search_engine/arguments.py:1-146),
so its scripts keep working; the last five rows are additions."""
from __future__ import annotations

import argparse

from ..utils.flag_table import flag_group

_MODES = ["static", "batch", "sequence"]

SEARCH_FLAGS = [
    # what is searched
    ("num_nodes", int, 1, "Number of Nodes."),
    ("num_gpus_per_node", int, 8, "Number of GPUs per node."),
    ("memory_constraint", int, 24, "Memory constraint of Galvatron (GB)"),
    ("search_space", ["full", "dp+tp", "dp+pp", "3d", "dp", "sdp", "tp", "pp"], "full"),
    ("sp_space", ["tp+sp", "tp", "sp"], "tp"),
    *[("disable_" + dim, int, 0) for dim in ("dp", "tp", "vtp", "pp", "sdp", "ckpt", "tp_consec")],
    ("max_tp_deg", int, 8), ("max_pp_deg", int, 8),
    ("fine_grained_mode", int, 1),
    # batch sizes
    ("min_bsz", int, 8), ("max_bsz", int, 10240), ("bsz_scale", int, 8),
    ("recommend_min_bsz", int, 0), ("settle_bsz", int, -1), ("settle_chunk", int, -1),
    # the runtime the plan is for
    ("default_dp_type", ["ddp", "zero2"], "ddp"),
    ("embed_sdp", int, 0),
    ("mixed_precision", ["fp32", "fp16", "bf16"], "bf16"),
    ("pipeline_type", ["gpipe", "pipedream_flush"], "gpipe"),
    ("sequence_parallel", "on", None),
    ("no_global_memory_buffer", "off:global_memory_buffer", None),
    ("no_async_grad_reduce", "off:async_grad_reduce", None),
    ("make-vocab-size-divisible-by", int, 128),
    # the model
    ("set_model_config_manually", int, 0), ("set_layernum_manually", int, 0), ("set_seqlen_manually", int, 0),
    # cost model
    ("use_pipeline_costmodel", int, 1), ("costmodel_coe", float, 1.0),
    ("time_profile_mode", _MODES, "static"), ("memory_profile_mode", _MODES, "static"),
    # files
    *[(name, str, None) for name in ("memory_profiling_path", "time_profiling_path", "allreduce_bandwidth_config_path",
                                     "p2p_bandwidth_config_path", "overlap_coe_path", "sp_time_path", "output_config_path")],
    ("log_dir", str, "logs"),
    ("parallel_search", "on", None), ("worker", int, 0),
    # additions
    ("bct_fct_coe", float, None, "Backward / forward time ratio of a layer (reference: fixed 2). Default: the value stored in the "
                                 "time profile under 'bct_fct_coe' if present, else 2."),
    ("check_cost_model", str, None, "'bsz,chunk,min_tp': print predicted stage memory and iteration time of every uniform strategy "
                                    "instead of searching (to compare the cost model with measured step times)."),
    ("explain_plan", str, None, "Path of a strategy JSON: print its predicted per-stage memory, per-stage time and step time "
                                "under the loaded profiles instead of searching."),
    ("memory_granularity_mb", int, 0, "Memory unit of the dynamic program in MB (0: 1 MB up to 32 Ki units, coarser above: a "
                                      "160 GB search then runs in 4 MB units)."),
    ("max_cp_deg", int, 1, "Also search a uniform zigzag context-parallel degree 1, 2, 4, ... up to this value (an extension: "
                           "the reference runs context parallelism but never searches it)."),
    ("memory_layout", ["engine", "fsdp"], "engine",
     "Model-state memory per rank: 'engine' = what this package's ZeRO engine keeps (full-size gradient buffer of --grad_dtype "
     "whatever the ZeRO stage, sharded optimizer slice), 'fsdp' = the reference's FSDP ratios."),
    ("context_mem_mb", int, 4096,
     "MB per rank on top of model states and profiled activations: gradient-reduction and loss transients, library "
     "workspaces (the reference's constant is 1024; Llama-7B peaks measured on 1, 2 and 8 B200s sit 2.9 GiB above states + "
     "activations)."),
    ("comm_impl", ["nccl", "fused"], "nccl",
     "Communication implementation of the run the plan is for: the peer-memory ZeRO engine ('fused') keeps its fp32 reduced "
     "gradient slice for the whole run (memory_layout engine)."),
    ("grad_dtype", ["fp32", "bf16"], "fp32", "Gradient-buffer precision of the run the plan is for (memory_layout engine)."),
    ("fused_comm_exposed", float, 1.0, "Exposed fraction of tensor/sequence-parallel communication of the fused kernels "
                                       "(1.0 = additive model)."),
]


def galvatron_search_args(parser: argparse.ArgumentParser) -> argparse.ArgumentParser:
    return flag_group(parser, "Galvatron Searching Arguments", SEARCH_FLAGS)
