"""Flags of the model profiler and the hardware profiler (names/defaults of the reference's
galvatron/core/profiler/arguments.py:1-85 and :88-194)."""
from __future__ import annotations

import argparse


def galvatron_profile_args(parser: argparse.ArgumentParser) -> argparse.ArgumentParser:
    g = parser.add_argument_group(title="Galvatron Profiling Arguments")
    g.add_argument("--profile_type", type=str, default="memory", choices=["memory", "computation"])
    g.add_argument("--set_model_config_manually", type=int, default=0)
    g.add_argument("--set_layernum_manually", type=int, default=1)
    g.add_argument("--set_seqlen_manually", type=int, default=0)
    g.add_argument("--profile_mode", type=str, default="static", choices=["static", "batch", "sequence"])
    g.add_argument("--profile_batch_size", type=int, default=None)
    g.add_argument("--profile_min_batch_size", type=int, default=None)
    g.add_argument("--profile_max_batch_size", type=int, default=None)
    g.add_argument("--profile_batch_size_step", type=int, default=1)
    g.add_argument("--profile_seq_length_list", type=str, default=None)
    g.add_argument("--profile_min_seq_length", type=int, default=None)
    g.add_argument("--profile_max_seq_length", type=int, default=None)
    g.add_argument("--profile_seq_length_step", type=int, default=128)
    g.add_argument("--layernum_min", type=int, default=1)
    g.add_argument("--layernum_max", type=int, default=2)
    g.add_argument("--max_tp_deg", type=int, default=8)
    g.add_argument("--profile_dp_type", type=str, default="zero3", choices=["zero3", "ddp"])
    g.add_argument("--mixed_precision", type=str, default="bf16", choices=["fp32", "fp16", "bf16"])
    g.add_argument("--use-flash-attn", action="store_true", dest="use_flash_attn")
    g.add_argument("--extra_args_str", type=str, default="")
    g.add_argument("--sequence_parallel", action="store_true")
    g.add_argument("--shape_order", type=str, default="SBH", choices=["SBH", "BSH"])
    g.add_argument("--make-vocab-size-divisible-by", type=int, default=128, dest="make_vocab_size_divisible_by")
    g.add_argument("--profile_dropout_prob", type=float, default=0.0,
                   help="Dropout probability of the profiled jobs (the reference fixes 0.1; here the profiles measure the "
                        "kernels alone by default and dropout is an element-wise add-on of the training run).")
    g.add_argument("--profile_iteration", type=int, default=1,
                   help="Computation profiling also times whole iterations to measure the backward / forward ratio.")
    g.add_argument("--in_process", type=int, default=1,
                   help="Measure single-GPU configurations inside this process instead of launching a job per point.")
    return parser


def galvatron_profile_hardware_args(parser: argparse.ArgumentParser) -> argparse.ArgumentParser:
    g = parser.add_argument_group(title="Galvatron Profiling Hardware Arguments")
    g.add_argument("--num_nodes", type=int, default=1)
    g.add_argument("--num_gpus_per_node", type=int, default=8)
    g.add_argument("--master_addr", type=str, default="$MASTER_ADDR")
    g.add_argument("--master_port", type=str, default="$MASTER_PORT")
    g.add_argument("--node_rank", type=str, default="$RANK")
    g.add_argument("--max_tp_size", type=int, default=8)
    g.add_argument("--envs", type=str, nargs="+", default=[])
    g.add_argument("--backend", type=str, default="native", choices=["native", "nccl", "torch"],
                   help="native: this package's own NVLink benchmark; nccl/torch: torch.distributed collectives.")
    g.add_argument("--nccl_test_dir", type=str, default="nccl-tests")
    g.add_argument("--mpi_path", type=str, default="/usr/local/mpi/")
    g.add_argument("--start_mb", type=int, default=16)
    g.add_argument("--end_mb", type=int, default=512)
    g.add_argument("--scale", type=int, default=2)
    g.add_argument("--hostfile", type=str, default="hostfile")
    g.add_argument("--avg_or_min_or_first", type=str, default="first", choices=["avg", "min", "first"])
    g.add_argument("--max_pp_deg", type=int, default=8)
    g.add_argument("--overlap_time_multiply", type=int, default=4)
    return parser
