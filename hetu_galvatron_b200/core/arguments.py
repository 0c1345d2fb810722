"""Command-line surface: ``initialize_galvatron(model_args, mode)`` + ``get_args()``.

Flag names and defaults follow the reference so its launch scripts keep working: the training group
(galvatron/core/runtime/arguments.py:1-215), the profile / hardware groups
(galvatron/core/profiler/arguments.py:1-194), the search group (search_engine/arguments.py:1-146) and the
Megatron flags its scripts pass (models/llama_hf/scripts/train_dist.sh:28-84). There is no Megatron global
state behind it: ``train_dist`` mode parses the flags, initialises ``torch.distributed`` (NCCL on GPUs, gloo
otherwise) and seeds the RNGs (reference: galvatron/core/arguments.py:8-31).
"""
from __future__ import annotations

import argparse
import os
from typing import Callable, Optional

_ARGS = None


def galvatron_training_args(parser: argparse.ArgumentParser, use_megatron: bool = True) -> argparse.ArgumentParser:
    g = parser.add_argument_group(title="Galvatron Training Arguments")
    g.add_argument("--set_model_config_manually", type=int, default=0)
    g.add_argument("--set_layernum_manually", type=int, default=0)
    g.add_argument("--set_seqlen_manually", type=int, default=0)
    g.add_argument("--initialize_on_meta", type=int, default=0, choices=[0, 1])
    g.add_argument("--global_train_batch_size", type=int, default=32)
    g.add_argument("--dropout_prob", type=float, default=0.1)
    g.add_argument("-e", "--epochs", type=int, default=10)
    g.add_argument("--adam_weight_decay", type=float, default=0.01)
    g.add_argument("--check_loss", type=int, default=0)
    g.add_argument("--profile", type=int, default=0)
    g.add_argument("--save_profiled_memory", type=int, default=0)
    g.add_argument("--profile_type", type=str, default="allocated", choices=["allocated", "reserved"])
    g.add_argument("--profile_mode", type=str, default="static", choices=["static", "batch", "sequence"])
    g.add_argument("--load_params", type=int, default=0)
    g.add_argument("--pp_deg", type=int, default=2, choices=[1, 2, 4, 8, 16, 32, 64, 128, 256, 512])
    g.add_argument("--global_cp_deg", type=int, default=1)
    g.add_argument("--cp_mode", type=str, default="zigzag", choices=["ring", "zigzag"])
    g.add_argument("--global_tp_deg", type=int, default=-1, choices=[-1, 1, 2, 4, 8, 16, 32])
    g.add_argument("--chunks", type=int, default=-1)
    g.add_argument("--global_tp_consec", type=int, default=-1, choices=[-1, 0, 1])
    g.add_argument("--sdp", type=int, default=0, choices=[0, 1])
    g.add_argument("--galvatron_config_path", type=str, default=None)
    g.add_argument("--global_checkpoint", type=int, default=0)
    g.add_argument("--mixed_precision", type=str, default="bf16", choices=["fp32", "fp16", "bf16"])
    g.add_argument("--loss_scale", type=float, default=None,
                   help="Constant loss scale (any precision). Unset: fp16 runs use the dynamic scaler, others none.")
    g.add_argument("--initial_loss_scale", type=float, default=2.0 ** 16, help="fp16: starting value of the dynamic loss scale.")
    g.add_argument("--min_loss_scale", type=float, default=1.0)
    g.add_argument("--loss_scale_window", type=int, default=1000, help="fp16: clean steps before the scale doubles.")
    g.add_argument("--hysteresis", type=int, default=2, help="fp16: overflowing steps tolerated before the scale halves.")
    g.add_argument("--pipeline_type", type=str, default="gpipe", choices=["gpipe", "pipedream_flush"])
    g.add_argument("--default_dp_type", type=str, default="ddp", choices=["ddp", "zero2", "zero3"])
    g.add_argument("--embed_sdp", type=int, default=0, choices=[0, 1])
    g.add_argument("--profile_forward", type=int, default=0, choices=[0, 1])
    g.add_argument("--save_profiled_iteration", type=int, default=0, choices=[0, 1],
                   help="Store the averaged time of whole iterations (forward + backward + optimizer) in the time profile.")
    g.add_argument("--allow_tf32", type=int, default=1, choices=[0, 1])
    g.add_argument("--exit_after_profiling", type=int, default=1, choices=[0, 1])
    g.add_argument("--shape_order", type=str, default="SBH", choices=["SBH", "BSH"])
    g.add_argument("--vocab_tp", type=int, default=1, choices=[1, 2, 4, 8, 16])
    g.add_argument("--vocab_cp", type=int, default=1)
    g.add_argument("--use-ulysses", action="store_true", dest="use_ulysses")
    g.add_argument("--no_async_grad_reduce", action="store_false", dest="async_grad_reduce")
    g.add_argument("--reduce_in_fp32", action="store_true")
    g.add_argument("--grad_dtype", type=str, default="fp32", choices=["fp32", "bf16"],
                   help="Precision of the flat gradient buffers micro-batches accumulate into (bf16 runs only; 2 instead "
                        "of 4 bytes per parameter on every rank, reductions still sum in fp32).")
    g.add_argument("--entropy_in_fp32", action="store_true")
    g.add_argument("--distributed_checkpoint", action="store_true", default=False)
    g.add_argument("--load_iteration", type=int, default=0)
    g.add_argument("--portable_optimizer_state", type=int, default=0, choices=[0, 1],
                   help="Also save fp32 master weights and Adam moments per block and parameter name, unsharded, so that "
                        "a run with another pipeline / data-parallel / ZeRO layout can resume (not in the reference).")
    g.add_argument("--allow_plan_change", type=int, default=0, choices=[0, 1],
                   help="Resume a distributed checkpoint under a plan that differs in anything but the tensor-parallel "
                        "degrees; needs a checkpoint saved with --portable_optimizer_state 1.")
    g.add_argument("--no-shared-storage", action="store_false", dest="shared_storage")
    # runtime extensions of this implementation
    g.add_argument("--comm_impl", type=str, default="nccl", choices=["nccl", "fused"],
                   help="Communication-bound paths: library collectives (nccl) or this package's peer-memory kernels (fused: "
                        "GEMM + collective, ZeRO gradient reduce-scatter / AdamW + parameter push / pull gathers, Ulysses "
                        "exchanges, context-parallel K/V pulls, relayout).")
    g.add_argument("--heartbeat_timeout_s", type=float, default=0.0,
                   help="> 0: every rank beats into the job's key-value store and every step runs between two health "
                        "checks (peer heartbeats, published failures, the device-side error word of bounded waits); a "
                        "rank that sees a failure prints it and leaves with exit code 3 instead of waiting for the "
                        "process-group timeout. 0 = off.")
    g.add_argument("--inject_rank_exit", type=str, default=None,
                   help="Host-side fault injection for recovery drills: 'RANK:ITER' makes that rank leave the job (exit "
                        "code 17) right before iteration ITER, between steps, with nothing of its own in flight.")
    g.add_argument("--random_dataset", type=int, default=0, choices=[0, 1],
                   help="Random-data programs: 1 draws batches from the family's random dataset (sentences of random length with "
                        "padding masks, BERT masking, images) through a torch DataLoader instead of dense synthetic tensors.")
    g.add_argument("--trace", type=str, default=None, help="Write a chrome-trace JSON of the profiled iterations here.")
    g.add_argument("--log_jsonl", type=str, default=None, help="Per-rank JSONL iteration log prefix.")
    # the subset of Megatron's training flags that the launch scripts use
    m = parser.add_argument_group(title="Training (Megatron-compatible names)")
    m.add_argument("--lr", type=float, default=1e-4)
    m.add_argument("--min-lr", type=float, default=0.0, dest="min_lr")
    m.add_argument("--lr-decay-style", type=str, default="linear", choices=["constant", "linear", "cosine", "inverse-square-root"], dest="lr_decay_style")
    m.add_argument("--lr-warmup-fraction", type=float, default=None, dest="lr_warmup_fraction")
    m.add_argument("--lr-warmup-iters", type=int, default=0, dest="lr_warmup_iters")
    m.add_argument("--lr-decay-iters", type=int, default=None, dest="lr_decay_iters")
    m.add_argument("--train-iters", type=int, default=None, dest="train_iters")
    m.add_argument("--weight-decay", type=float, default=0.01, dest="weight_decay")
    m.add_argument("--adam-beta1", type=float, default=0.9, dest="adam_beta1")
    m.add_argument("--adam-beta2", type=float, default=0.999, dest="adam_beta2")
    m.add_argument("--adam-eps", type=float, default=1e-8, dest="adam_eps")
    m.add_argument("--init-method-std", type=float, default=0.02, dest="init_method_std")
    m.add_argument("--clip-grad", type=float, default=1.0, dest="clip_grad")
    m.add_argument("--seed", type=int, default=1234)
    m.add_argument("--data-path", nargs="*", default=None, dest="data_path")
    m.add_argument("--split", type=str, default="969,30,1")
    m.add_argument("--tokenizer-type", type=str, default=None, dest="tokenizer_type")
    m.add_argument("--tokenizer-model", type=str, default=None, dest="tokenizer_model")
    m.add_argument("--save", type=str, default=None)
    m.add_argument("--save-interval", type=int, default=None, dest="save_interval")
    m.add_argument("--load", type=str, default=None)
    m.add_argument("--sequence-parallel", action="store_true", dest="sequence_parallel")
    m.add_argument("--use-flash-attn", action="store_true", dest="use_flash_attn")
    m.add_argument("--distributed-backend", type=str, default=None, dest="distributed_backend")
    m.add_argument("--distributed-timeout-minutes", type=int, default=10, dest="distributed_timeout_minutes")
    m.add_argument("--local-rank", "--local_rank", type=int, default=int(os.environ.get("LOCAL_RANK", "0")), dest="local_rank")
    m.add_argument("--gpu_id", type=int, default=0)
    m.add_argument("--make-vocab-size-divisible-by", type=int, default=128, dest="make_vocab_size_divisible_by")
    m.add_argument("--eval-iters", type=int, default=0, dest="eval_iters")
    m.add_argument("--eval-interval", type=int, default=1000, dest="eval_interval")
    return parser


def _parse(providers, argv=None) -> argparse.Namespace:
    parser = argparse.ArgumentParser(description="Galvatron Arguments", allow_abbrev=False)
    for p in providers:
        if p is not None:
            parser = p(parser) or parser
    args, _unknown = parser.parse_known_args(argv)
    return args


def initialize_galvatron(model_args: Optional[Callable] = None, mode: str = "train_dist", argv=None):
    """Parse the flags of ``mode`` (+ the model's own flags) and, for ``train_dist``, start the process group.

    Modes: ``train_dist`` (hybrid-parallel training), ``train`` (single device), ``profile`` (model profiler),
    ``search`` (search engine), ``profile_hardware`` (hardware profiler)."""
    global _ARGS
    from ..profiler.arguments import galvatron_profile_args, galvatron_profile_hardware_args
    from ..search.arguments import galvatron_search_args

    if mode in ("train_dist", "train"):
        args = _parse([galvatron_training_args, model_args], argv)
    elif mode == "profile":
        args = _parse([galvatron_profile_args, model_args], argv)
    elif mode == "search":
        args = _parse([galvatron_search_args, model_args], argv)
    elif mode == "profile_hardware":
        args = _parse([galvatron_profile_hardware_args, model_args], argv)
    else:
        raise ValueError("unknown mode %r" % mode)
    args.galvatron_mode = mode
    if mode == "train_dist":
        _init_distributed(args)
    if mode in ("train_dist", "train"):
        import torch

        if getattr(args, "allow_tf32", 1):
            torch.backends.cuda.matmul.allow_tf32 = True
            torch.backends.cudnn.allow_tf32 = True
        from ..utils.training_utils import set_seed

        set_seed(args.seed)
    _ARGS = args
    return args


def _init_distributed(args) -> None:
    import datetime

    import torch
    import torch.distributed as dist

    args.rank = int(os.environ.get("RANK", "0"))
    args.world_size = int(os.environ.get("WORLD_SIZE", "1"))
    args.local_rank = int(os.environ.get("LOCAL_RANK", args.local_rank))
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(args.local_rank)
    backend = args.distributed_backend or ("nccl" if use_cuda else "gloo")
    if args.world_size > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        dist.init_process_group(backend=backend, timeout=datetime.timedelta(minutes=args.distributed_timeout_minutes))


def get_args():
    if _ARGS is None:
        raise RuntimeError("initialize_galvatron() has not been called")
    return _ARGS


def set_args(args) -> None:
    global _ARGS
    _ARGS = args


def __getattr__(name: str):
    """The profile / hardware-profile / search argument groups are importable from here too, as in the reference
    (galvatron/core/arguments.py:4-6); resolved on first use to keep this module free of import cycles."""
    if name in ("galvatron_profile_args", "galvatron_profile_hardware_args"):
        from ..profiler import arguments as _p
        return getattr(_p, name)
    if name == "galvatron_search_args":
        from ..search.arguments import galvatron_search_args
        return galvatron_search_args
    raise AttributeError("module %r has no attribute %r" % (__name__, name))
