"""Flags of the model profiler and the hardware profiler. Names and defaults are the reference's
(galvatron/core/profiler/arguments.py:1-85 and :88-194); the rows marked as additions are new."""
from __future__ import annotations

import argparse

from ..utils.flag_table import flag_group

MODEL_PROFILE_FLAGS = [
    ("profile_type", ["memory", "computation"], "memory"),
    ("profile_mode", ["static", "batch", "sequence"], "static"),
    # the grid of measured points
    ("profile_batch_size", int, None), ("profile_min_batch_size", int, None), ("profile_max_batch_size", int, None),
    ("profile_batch_size_step", int, 1),
    ("profile_seq_length_list", str, None), ("profile_min_seq_length", int, None), ("profile_max_seq_length", int, None),
    ("profile_seq_length_step", int, 128),
    ("layernum_min", int, 1), ("layernum_max", int, 2),
    ("max_tp_deg", int, 8),
    # how the measured jobs run
    ("profile_dp_type", ["zero3", "ddp"], "zero3"),
    ("mixed_precision", ["fp32", "fp16", "bf16"], "bf16"),
    ("use-flash-attn", "on", None),
    ("sequence_parallel", "on", None),
    ("shape_order", ["SBH", "BSH"], "SBH"),
    ("make-vocab-size-divisible-by", int, 128),
    ("extra_args_str", str, ""),
    ("set_model_config_manually", int, 0), ("set_layernum_manually", int, 1), ("set_seqlen_manually", int, 0),
    # additions
    ("profile_dropout_prob", float, 0.0, "Dropout probability of the profiled jobs (the reference fixes 0.1; here the profiles "
                                         "measure the kernels alone by default and dropout is an element-wise add-on of the "
                                         "training run)."),
    ("profile_iteration", int, 1, "Computation profiling also times whole iterations to measure the backward / forward ratio."),
    ("memory_layout", ["engine", "fsdp"], "engine",
     "How measured model states are turned into a parameter size: 'engine' inverts this package's ZeRO-engine layout "
     "(search/cost_model.engine_state_ratio, fp32 gradient buffers), 'fsdp' assumes ideal sharding as the reference does."),
    ("process_only", int, 0, "Skip the measurements and post-process the raw numbers already in the profile file."),
    ("in_process", int, 1, "Measure single-GPU configurations inside this process instead of launching a job per point."),
]

HARDWARE_PROFILE_FLAGS = [
    ("num_nodes", int, 1), ("num_gpus_per_node", int, 8),
    ("master_addr", str, "$MASTER_ADDR"), ("master_port", str, "$MASTER_PORT"), ("node_rank", str, "$RANK"),
    ("max_tp_size", int, 8), ("max_pp_deg", int, 8),
    ("backend", ["native", "nccl", "torch"], "native",
     "native: this package's own NVLink benchmark; nccl/torch: torch.distributed collectives."),
    ("start_mb", int, 16), ("end_mb", int, 512), ("scale", int, 2),
    ("avg_or_min_or_first", ["avg", "min", "first"], "first"),
    ("overlap_time_multiply", int, 4),
    # kept for script compatibility with the reference's nccl-tests / mpirun driver; unused by the in-job measurements
    ("nccl_test_dir", str, "nccl-tests"), ("mpi_path", str, "/usr/local/mpi/"), ("hostfile", str, "hostfile"),
]


def galvatron_profile_args(parser: argparse.ArgumentParser) -> argparse.ArgumentParser:
    return flag_group(parser, "Galvatron Profiling Arguments", MODEL_PROFILE_FLAGS)


def galvatron_profile_hardware_args(parser: argparse.ArgumentParser) -> argparse.ArgumentParser:
    flag_group(parser, "Galvatron Profiling Hardware Arguments", HARDWARE_PROFILE_FLAGS)
    parser.add_argument("--envs", type=str, nargs="+", default=[])
    return parser
