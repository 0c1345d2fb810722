"""Argument bundles of the cost models.

Five dataclasses group what the cost models need: the layer's shape, training options, the parallel set-up being
priced, the model profile and the hardware profile. Class and field names are those of the reference's
galvatron/core/search_engine/cost_model_args.py:6-49, because the DP driver and user code construct them by keyword;
the defaults here are what was measured for one Llama-7B layer (sequence 4096, bf16) on an 8 x B200 NVSwitch node, so a
cost model built without profiles still answers for that machine. The search engine always overrides them from the
profile files.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Optional, Union

import numpy as np

# all-reduce bus bandwidth (GB/s) measured on 8 x B200 for groups of 8 / 4 / 2 ranks and pipeline send/recv bandwidth
_B200_ALLREDUCE_GBS = {"8": 606.7, "4_0": 549.1, "4_1": 548.8, "2_0": 469.9, "2_1": 469.3}
_B200_P2P_GBS = {2: 513.1, 4: 276.1, 8: 304.1}


def _coefficients(bandwidth: dict) -> dict:
    """ms per MB = 1 / (GB/s), the unit the time model multiplies message sizes (MB) with."""
    return {k: 1.0 / v for k, v in bandwidth.items()}


@dataclass
class ModelArgs:
    """One layer type of the model."""
    parameter_size: float = 48          # MB of fp32 parameters of one layer (before tensor-parallel sharding)
    seq_length: int = 1024
    hidden_size: int = 4096
    layer_num: int = 16                 # layers of this type in the model


@dataclass
class TrainArgs:
    mixed_precision: bool = False       # bf16 / fp16 compute: halves message sizes, changes the ZeRO ratios
    checkpoint: bool = False
    async_grad_reduce: bool = True      # gradients reduced once per step (full-size gradients live during accumulation)
    pytorch_context_mem: int = 1024     # MB per rank outside the model: CUDA context, NCCL buffers, workspaces
    # "fsdp": the reference's ZeRO ratios (gradients and parameters freed as FSDP frees them); "engine": what this
    # package's ZeRO engine keeps per rank (cost_model.engine_state_ratio), with gradient buffers of grad_bytes
    memory_layout: str = "fsdp"
    grad_bytes: int = 4
    # engine layout only: the data-parallel engine runs on the peer-memory kernels, which keep the fp32 reduced gradient
    # slice (4 bytes per parameter over the sharding degree) for the whole run instead of allocating it per step
    fused_engine: bool = False


@dataclass
class ParallelArgs:
    use_zero2_for_dp: bool = False      # the plan's default data-parallel type is ZeRO-2 instead of DDP
    disable_vtp: bool = False           # price only vocab-tp = 1 for embedding and head
    sequence_parallel: bool = False     # Megatron-SP inside tensor-parallel groups
    sp_space: str = "sp+tp"             # "tp": bandwidth model of TP traffic; "tp+sp": latency tables (TP and Ulysses)
    pipeline_type: str = "gpipe"
    optimal_chunk_func: Optional[Callable] = None     # (local_bsz, strategy, mbsz, min_tp) -> micro-batch count
    chunks: Optional[int] = None        # fixed micro-batch count (None: ask optimal_chunk_func)
    # Uniform context-parallel degree around the searched sub-world (an extension, search/context_parallel.py): the
    # context-parallel ranks replicate the weights, so ZeRO shards and gradient reduction span cp_size x dp ranks.
    cp_size: int = 1


@dataclass
class ProfileModelArgs:
    """What the model profiler measured (defaults: Llama-7B layer, sequence 4096, Megatron-SP, B200)."""
    # activation MB per sample at each tensor-parallel degree; "checkpoint": what a recomputed layer keeps
    tp_activation_per_bsz_dict: dict = field(default_factory=lambda: {1: 366.0, 2: 214.3, 4: 107.1, 8: 53.6, "checkpoint": 48.3})
    # embedding + head + final norm: model states (MB) and activation (MB per sample); scalars or {vocab_tp: MB} tables
    other_memory_pp_off: dict = field(default_factory=lambda: {"model_states": 6501.0, "activation": 322.8})
    other_memory_pp_on: dict = field(default_factory=lambda: {
        "first_stage": {"model_states": 704.5, "activation": 384.5},
        "last_stage": {"model_states": 704.5, "activation": 408.6}})
    # forward ms per layer and sample, or the (slope, intercept) of a fit over the batch size
    forward_computation_time: Optional[Union[float, np.ndarray]] = 1.762
    other_time_profiled: Optional[Union[float, np.ndarray]] = 0.893
    # optimizer step (+ zero_grad) of one un-sharded layer, ms per training step (0: folded into bct_fct_coe, as the
    # reference does); paid once per step whatever the micro-batch count, divided by the tensor-parallel degree and,
    # under ZeRO, by the sharding degree
    optimizer_time: float = 0.0


@dataclass
class ProfileHardwareArgs:
    """What the hardware profiler measured (defaults: one 8 x B200 NVSwitch node)."""
    bct_fct_coe: float = 2              # backward / forward time; the model profiler measures 2.35 for Llama-7B
    extra_overhead: float = 0           # ms added to every layer that has data-parallel traffic
    comm_coe_dict: dict = field(default_factory=lambda: dict(_coefficients(_B200_ALLREDUCE_GBS), **{"1": 0}))
    dp_overlap_coe: float = 1.3         # slow-down of gradient traffic while backward compute runs
    bct_overlap_coe: float = 1.3        # slow-down of backward compute while gradient traffic runs
    p2p_comm_coe_dict: dict = field(default_factory=lambda: _coefficients(_B200_P2P_GBS))
    allreduce_dict: dict = field(default_factory=dict)    # {group size: {bytes: ms, "popt": (slope, intercept)}}
    all2all_dict: dict = field(default_factory=dict)
    costmodel_coe: float = 1.0
    # Measured exposed fraction of tensor/sequence-parallel communication when it is fused into the GEMM that
    # produces/consumes it (1.0 = nothing hidden, the additive model of a library-collective runtime).
    fused_comm_exposed: float = 1.0
