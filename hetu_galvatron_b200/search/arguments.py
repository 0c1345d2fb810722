"""Search-engine command-line flags (same names and defaults as the reference's
galvatron/core/search_engine/arguments.py:1-146)."""
from __future__ import annotations

import argparse


def galvatron_search_args(parser: argparse.ArgumentParser) -> argparse.ArgumentParser:
    g = parser.add_argument_group(title="Galvatron Searching Arguments")
    g.add_argument("--set_model_config_manually", type=int, default=0)
    g.add_argument("--set_layernum_manually", type=int, default=0)
    g.add_argument("--set_seqlen_manually", type=int, default=0)
    g.add_argument("--num_nodes", type=int, default=1, help="Number of Nodes.")
    g.add_argument("--num_gpus_per_node", type=int, default=8, help="Number of GPUs per node.")
    g.add_argument("--memory_constraint", type=int, default=24, help="Memory constraint of Galvatron (GB)")
    g.add_argument("--min_bsz", type=int, default=8)
    g.add_argument("--max_bsz", type=int, default=10240)
    g.add_argument("--recommend_min_bsz", type=int, default=0)
    g.add_argument("--settle_bsz", type=int, default=-1)
    g.add_argument("--settle_chunk", type=int, default=-1)
    g.add_argument("--bsz_scale", type=int, default=8)
    g.add_argument("--search_space", type=str, default="full", choices=["full", "dp+tp", "dp+pp", "3d", "dp", "sdp", "tp", "pp"])
    g.add_argument("--sp_space", type=str, default="tp", choices=["tp+sp", "tp", "sp"])
    for name in ("dp", "tp", "vtp", "pp", "sdp", "ckpt", "tp_consec"):
        g.add_argument("--disable_%s" % name, type=int, default=0)
    g.add_argument("--max_tp_deg", type=int, default=8)
    g.add_argument("--max_pp_deg", type=int, default=8)
    g.add_argument("--default_dp_type", type=str, default="ddp", choices=["ddp", "zero2"])
    g.add_argument("--embed_sdp", type=int, default=0)
    g.add_argument("--mixed_precision", type=str, default="bf16", choices=["fp32", "fp16", "bf16"])
    g.add_argument("--pipeline_type", type=str, default="gpipe", choices=["gpipe", "pipedream_flush"])
    g.add_argument("--use_pipeline_costmodel", type=int, default=1)
    g.add_argument("--costmodel_coe", type=float, default=1.0)
    g.add_argument("--sequence_parallel", action="store_true")
    g.add_argument("--no_global_memory_buffer", action="store_false", dest="global_memory_buffer")
    g.add_argument("--no_async_grad_reduce", action="store_false", dest="async_grad_reduce")
    g.add_argument("--memory_profiling_path", type=str, default=None)
    g.add_argument("--time_profiling_path", type=str, default=None)
    g.add_argument("--allreduce_bandwidth_config_path", type=str, default=None)
    g.add_argument("--p2p_bandwidth_config_path", type=str, default=None)
    g.add_argument("--overlap_coe_path", type=str, default=None)
    g.add_argument("--sp_time_path", type=str, default=None)
    g.add_argument("--output_config_path", type=str, default=None)
    g.add_argument("--make-vocab-size-divisible-by", type=int, default=128)
    g.add_argument("--fine_grained_mode", type=int, default=1)
    g.add_argument("--time_profile_mode", type=str, default="static", choices=["static", "batch", "sequence"])
    g.add_argument("--memory_profile_mode", type=str, default="static", choices=["static", "batch", "sequence"])
    g.add_argument("--parallel_search", action="store_true")
    g.add_argument("--worker", type=int, default=0)
    g.add_argument("--log_dir", type=str, default="logs")
    g.add_argument("--bct_fct_coe", type=float, default=None,
                   help="Backward / forward time ratio of a layer (reference: fixed 2). Default: the value stored in the "
                        "time profile under 'bct_fct_coe' if present, else 2.")
    g.add_argument("--check_cost_model", type=str, default=None,
                   help="'bsz,chunk,min_tp': print predicted stage memory and iteration time of every uniform strategy "
                        "instead of searching (to compare the cost model with measured step times).")
    g.add_argument("--memory_granularity_mb", type=int, default=0,
                   help="Memory unit of the dynamic program in MB (0: 1 MB up to 32 Ki units, coarser above: a 160 GB "
                        "search then runs in 4 MB units).")
    g.add_argument("--max_cp_deg", type=int, default=1,
                   help="Also search a uniform zigzag context-parallel degree 1, 2, 4, ... up to this value "
                        "(an extension: the reference runs context parallelism but never searches it).")
    g.add_argument("--fused_comm_exposed", type=float, default=1.0,
                   help="Exposed fraction of tensor/sequence-parallel communication of the fused kernels (1.0 = additive model).")
    return parser
