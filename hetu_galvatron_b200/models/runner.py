"""The four per-family programs of the reference's model zoo, implemented once and parameterised by family:

* ``train_dist``          hybrid-parallel training on a dataset or random tokens (models/*/train_dist.py)
* ``train_dist_random``   the same loop on synthetic data, used for profiling (models/*/train_dist_random.py)
* ``profiler``            model profiler entry (models/*/profiler.py)
* ``search_dist``         search-engine entry (models/*/search_dist.py)

Each family module under ``models/<family>_programs`` only binds the family name.
"""
from __future__ import annotations

import os
import sys

import torch

from .arguments import base_family


def _dtype(args):
    return {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}[args.mixed_precision]


def build_model(family: str, args):
    """args -> (GalvatronModel, ModelConfig, HybridPlan): GLOBAL flags or --galvatron_config_path JSON."""
    import torch.distributed as dist

    from ..core.hybrid_model import construct_hybrid_parallel_model
    from ..core.plan import HybridPlan
    from .arguments import config_from_args

    world = dist.get_world_size() if dist.is_initialized() else 1
    device = torch.device("cuda", args.local_rank) if torch.cuda.is_available() else torch.device("cpu")
    cfg, specs = config_from_args(family, args, _dtype(args))
    n_layers = len([s for s in specs if s.layer_index is not None])
    if base_family(family) in ("vit", "swin") and (getattr(args, "sequence_parallel", False) or getattr(args, "use_ulysses", False)):
        # vision models keep whole token grids per rank: 197 / 257 tokens do not split over ranks and window
        # partition / patch merging need the full grid (the reference forces the same,
        # galvatron/models/vit_hf/ViTModel_hybrid_parallel.py:79-80)
        if not dist.is_initialized() or dist.get_rank() == 0:
            print("note: sequence parallelism is not used for the %s family; running tensor parallel without it" % family)
        args.sequence_parallel, args.use_ulysses = False, False
    if args.galvatron_config_path not in (None, "None"):
        plan = HybridPlan.from_json(args.galvatron_config_path, n_layers, sequence_parallel=args.sequence_parallel,
                                    pipeline_type=args.pipeline_type, default_dp_type=args.default_dp_type,
                                    embed_sdp=args.embed_sdp)
        args.global_train_batch_size, args.chunks, args.pp_deg = plan.global_bsz, plan.chunks, plan.pp_deg
        args.vocab_tp, args.vocab_sp, args.vocab_cp = plan.vocab_tp, plan.vocab_sp, plan.vocab_cp
    else:
        plan = HybridPlan.from_global(n_layers, world, pp_deg=args.pp_deg, global_tp_deg=args.global_tp_deg,
                                      global_cp_deg=args.global_cp_deg, sdp=args.sdp, global_checkpoint=args.global_checkpoint,
                                      use_ulysses=args.use_ulysses, vocab_tp=args.vocab_tp, vocab_cp=args.vocab_cp,
                                      chunks=args.chunks, global_bsz=args.global_train_batch_size,
                                      pipeline_type=args.pipeline_type, default_dp_type=args.default_dp_type,
                                      embed_sdp=args.embed_sdp, sequence_parallel=args.sequence_parallel)
        args.chunks = plan.chunks
    import contextlib

    from .transformer import deferred_init

    # --initialize_on_meta 1 with --load: the weights come from the checkpoint, so they are created without values
    defer = bool(getattr(args, "initialize_on_meta", 0)) and bool(getattr(args, "load", None))
    with (deferred_init() if defer else contextlib.nullcontext()):
        model = construct_hybrid_parallel_model(cfg, plan, specs, device, impl=args.comm_impl,
                                                async_grad_reduce=args.async_grad_reduce, reduce_in_fp32=args.reduce_in_fp32,
                                                grad_dtype=torch.bfloat16 if getattr(args, "grad_dtype", "fp32") == "bf16"
                                                and _dtype(args) == torch.bfloat16 else torch.float32,
                                                verbose=True)
    if getattr(args, "load", None):
        from ..core.checkpoint import load_model
        load_model(model, args.load, family, iteration=args.load_iteration if args.distributed_checkpoint else None,
                   allow_plan_change=bool(getattr(args, "allow_plan_change", 0)))
    return model, cfg, plan


def program_dir(family: str) -> str:
    """Directory whose ``configs/`` holds the family's profiles and searched plans. The ``*_fa`` names share the
    directory (and so the profiles) of their base family: they run the same model definition and kernels."""
    fam = base_family(family)
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), fam + "_programs")


def get_runtime_profiler(args, path, cfg, family, start_iter=10, end_iter=20):
    from ..profiler.runtime_profiler import RuntimeProfiler
    from . import model_name_and_layer_configs

    name, layer_cfgs = model_name_and_layer_configs(family, cfg, args)
    prof = RuntimeProfiler(args, path=path, model_name=name, log_path=getattr(args, "log_jsonl", None))
    prof.set_profiler_dist(path, layer_cfgs, name, start_iter=start_iter, end_iter=end_iter)
    prof.tokens_per_iter = args.global_train_batch_size * cfg.seq_length
    return prof


def _random_dataset_iterator(family, args, cfg, plan, model, iters: int):
    """Batches of this rank from the family's random dataset (models/dataloader.py), moved to the model's device; the
    way the reference's ``train_dist_random.py`` programs feed their models (e.g. models/llama_hf/train_dist_random.py:40-52)."""
    from types import SimpleNamespace

    from ..utils.training_utils import distributed_dataloader
    from .dataloader import random_dataset

    ns = SimpleNamespace(vocab_size=cfg.vocab_size, seq_length=cfg.seq_length, encoder_seq_length=cfg.seq_length,
                         decoder_seq_length=getattr(cfg, "decoder_seq_length", None), image_size=cfg.image_size,
                         num_channels=cfg.num_channels, num_labels=cfg.num_labels, seed=args.seed)
    ds, collate = random_dataset(family, ns, None, max(plan.global_bsz * max(iters, 1), plan.global_bsz))
    loader = distributed_dataloader(ds, plan.global_bsz, shuffle=False, collate_fn=collate, model=model)

    def move(x):
        if isinstance(x, dict):
            return {k: move(v) for k, v in x.items()}
        x = x.to(model.device, non_blocking=True)
        return x.to(cfg.dtype) if x.is_floating_point() else x

    def batches():
        while True:
            for b in loader:
                yield tuple(move(t) for t in b)

    return batches()


def train(family: str, random_data: bool = True, argv=None, single_device: bool = False) -> None:
    """``single_device``: the reference's plain ``train.py`` (galvatron/models/bert_hf/train.py:32-85): no process group,
    the whole model on one device (pp = tp = 1), time / memory profiled by the single-device profiler set-up."""
    from ..core.arguments import initialize_galvatron
    from ..core.optimizer import get_optimizer_and_param_scheduler
    from ..utils.training_utils import print_loss
    from . import synthetic_batch
    from .arguments import make_model_args

    args = initialize_galvatron(make_model_args(family), mode="train" if single_device else "train_dist", argv=argv)
    if single_device:
        args.pp_deg, args.global_tp_deg, args.global_cp_deg, args.vocab_tp, args.sdp, args.use_ulysses = 1, 1, 1, 1, 0, False
        args.galvatron_config_path = None
    model, cfg, plan = build_model(family, args)
    optimizer, scheduler = get_optimizer_and_param_scheduler(model, args)
    path = program_dir(family)
    profiler = get_runtime_profiler(args, path, cfg, family)
    if single_device:
        profiler.set_profiler_single()
    profiler.profile_memory(0, "After creating model")
    iters = args.train_iters or 25
    tracer = None
    if getattr(args, "trace", None):
        from ..utils.trace import enable_tracing
        tracer = enable_tracing(torch.distributed.get_rank() if torch.distributed.is_initialized() else 0)
    data_iter = None
    if not random_data and args.data_path:
        from ..core.dataloader import build_token_iterator
        data_iter = build_token_iterator(args, cfg, model)
    if data_iter is None and getattr(args, "random_dataset", 0):
        data_iter = _random_dataset_iterator(family, args, cfg, plan, model, iters)
    # validation (Megatron flags --eval-iters / --eval-interval): forward-only passes over the validation split of
    # --data-path, or over synthetic batches from a seed range the training batches never use
    eval_iters, eval_interval = int(getattr(args, "eval_iters", 0) or 0), int(getattr(args, "eval_interval", 0) or 0)
    valid_iter = None
    if eval_iters > 0 and data_iter is not None:
        from ..core.dataloader import build_token_iterator
        valid_iter = build_token_iterator(args, cfg, model, which=1)

    def evaluate(it: int):
        import math
        total, seen = 0.0, 0
        for k in range(eval_iters):
            if valid_iter is not None:
                vb = next(valid_iter)
            else:
                vb = synthetic_batch(family, cfg, plan.global_bsz, seed=args.seed + 1_000_003 + k, device=model.device)
                vb = tuple(t[lo:hi] if torch.is_tensor(t) else {kk: v[lo:hi] for kk, v in t.items()} for t in vb)
            vl = model.mean_loss_over_ranks(model.forward_backward(vb, it, None, forward_only=True))
            if vl is not None:
                total, seen = total + float(vl), seen + 1
        if seen:
            mean = total / seen
            print(" validation loss at iteration %d | lm loss value: %.6E | lm loss PPL: %.6E |" % (
                it, mean, math.exp(min(mean, 20.0))), flush=True)
            return mean
        return None

    # explicit in both directions: the model profiler runs several jobs in one process
    torch.set_grad_enabled(not getattr(args, "profile_forward", 0))
    lo, hi = model.batch_slice()
    start = args.load_iteration if getattr(args, "distributed_checkpoint", False) else 0
    heartbeat, inject = _start_heartbeat(args), _parse_injection(getattr(args, "inject_rank_exit", None))
    for it in range(start, iters):
        if inject is not None and inject == (torch.distributed.get_rank() if torch.distributed.is_initialized() else 0, it):
            sys.stdout.flush()
            os._exit(17)            # drill: this rank is lost between two steps
        if data_iter is not None:
            batch = next(data_iter)
        else:
            batch = synthetic_batch(family, cfg, plan.global_bsz, seed=args.seed + it, device=model.device)
            batch = tuple(t[lo:hi] if torch.is_tensor(t) else {k: v[lo:hi] for k, v in t.items()} for t in batch)
        profiler.profile_time_start(it)
        profiler.profile_memory(it, "Before Forward")

        def one_step(batch=batch, it=it):
            loss = model.forward_backward(batch, it, None, forward_only=bool(getattr(args, "profile_forward", 0)))
            profiler.profile_memory(it, "After Backward")
            norm = None
            if not getattr(args, "profile_forward", 0):
                profiler.profile_optimizer_start()
                norm = optimizer.step()
                if not optimizer.skipped_last_step:     # an overflowing fp16 step changes neither weights nor schedule
                    scheduler.step(increment=args.global_train_batch_size)
                optimizer.zero_grad()
                profiler.profile_optimizer_end(it)
            return loss, norm

        if heartbeat is None:
            loss, norm = one_step()
        else:
            from ..core.failure import RankFailure, guarded_step
            try:
                loss, norm = guarded_step(one_step, heartbeat, check_device=model.device.type == "cuda")
            except RankFailure as failure:
                _leave_after_failure(failure, heartbeat, it)
        profiler.profile_memory(it, "After optimizer_step")
        if optimizer.skipped_last_step and (not torch.distributed.is_initialized() or torch.distributed.get_rank() == 0):
            print("(Iteration %d): gradient overflow, step skipped; loss scale now %g" % (it, optimizer.loss_scale), flush=True)
        if args.check_loss or not args.profile:
            print_loss(args, model.mean_loss_over_ranks(loss), 0, it)
        profiler.post_profile_memory(it)
        profiler.profile_time_end(it, model.mean_loss_over_ranks(loss), optimizer.lr, norm)
        if tracer is not None and it == min(iters - 1, 12):
            print("trace written to", tracer.dump(args.trace), flush=True)
            tracer.enabled = False
        if eval_iters > 0 and eval_interval > 0 and (it + 1) % eval_interval == 0:
            evaluate(it + 1)
        if args.save and args.save_interval and (it + 1) % args.save_interval == 0:
            from ..core.checkpoint import save_model
            save_model(model, args.save, family, it + 1, optimizer=optimizer,
                       portable_optimizer=bool(getattr(args, "portable_optimizer_state", 0)))


def _parse_injection(text):
    if not text:
        return None
    rank, it = str(text).split(":")
    return int(rank), int(it)


def _start_heartbeat(args):
    """``--heartbeat_timeout_s T``: liveness of every rank through the process group's own key-value store."""
    timeout = float(getattr(args, "heartbeat_timeout_s", 0.0) or 0.0)
    dist = torch.distributed
    if timeout <= 0 or not dist.is_initialized() or dist.get_world_size() < 2:
        return None
    from ..core.failure import Heartbeat

    store = dist.PrefixStore("gv_heartbeat", dist.distributed_c10d._get_default_store())
    return Heartbeat(store, dist.get_rank(), dist.get_world_size(), interval_s=min(0.5, timeout / 4), timeout_s=timeout).start()


def _leave_after_failure(failure, heartbeat, iteration: int) -> None:
    """A peer is gone (or a device wait of this rank gave up): say so once and leave without touching the process group
    again -- its collectives can no longer complete. The job is restarted from its last checkpoint, under a plan
    searched for the surviving ranks if need be (``core.failure.replan_for_world_size``)."""
    print("RANK FAILURE at iteration %d on rank %d: %s" % (iteration, heartbeat.rank, failure), flush=True)
    heartbeat.stop(leaving=True)
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(3)


def profile(family: str, argv=None) -> None:
    from ..core.arguments import initialize_galvatron
    from ..profiler.model_profiler import ModelProfiler
    from .arguments import layernum_arg_names, make_model_args

    from . import model_name_and_layer_configs
    from .arguments import config_from_args

    args = initialize_galvatron(make_model_args(family), mode="profile", argv=argv)
    cfg, _ = config_from_args(family, args, torch.bfloat16)
    if args.profile_mode != "sequence" and base_family(family) not in ("vit", "swin"):
        # the measured jobs run at the profile length (--profile_seq_length_list, else --seq_length, else the model's
        # own); the profile file is named after it
        if args.profile_seq_length_list:
            lengths = [int(v) for v in str(args.profile_seq_length_list).split(",")]
            cfg.seq_length = lengths[0]
            if base_family(family) == "t5" and len(lengths) > 1 and lengths[1] != lengths[0]:
                cfg.decoder_seq_length = lengths[1]           # one length per layer type: encoder, decoder
        elif getattr(args, "seq_length", None):
            cfg.seq_length = args.seq_length
        args.seq_length = cfg.seq_length
    name, _ = model_name_and_layer_configs(family, cfg, args)
    if base_family(family) == "vit":
        args.seq_length = cfg.seq_length       # fixed by image and patch size
    if base_family(family) in ("vit", "swin"):
        # flags left at their defaults take the model size's values (the profiler derives sequence lengths from them)
        for flag, value in (("image_size", cfg.image_size), ("patch_size", cfg.patch_size), ("depths", getattr(cfg, "depths", None)),
                            ("embed_dim", getattr(cfg, "embed_dim", None)), ("window_size", getattr(cfg, "window_size", None))):
            if hasattr(args, flag) and getattr(args, flag) is None and value is not None:
                setattr(args, flag, list(value) if isinstance(value, (list, tuple)) else value)
    prof = ModelProfiler(args)
    prof.family = family
    prof.set_profiler_launcher(program_dir(family), layernum_arg_names(family), name,
                               seqlen_arg_names=(["encoder_seq_length", "decoder_seq_length"] if base_family(family) == "t5" else
                                                 None if base_family(family) not in ("vit", "swin") else []),
                               layernum_listed=family == "swin")
    if getattr(args, "process_only", 0):
        prof.process_profiled_data()
        return
    prof.launch_profiling_scripts()
    dist = torch.distributed
    if dist.is_initialized():            # the profiler ran as one rank of a job (in-process points): one writer
        dist.barrier()
        if dist.get_rank() == 0:
            prof.process_profiled_data()
        dist.barrier()
        dist.destroy_process_group()
    else:
        prof.process_profiled_data()


def search(family: str, argv=None):
    from ..core.arguments import initialize_galvatron
    from ..search import GalvatronSearchEngine
    from . import model_name_and_layer_configs
    from .arguments import config_from_args, make_model_args

    args = initialize_galvatron(make_model_args(family), mode="search", argv=argv)
    args.local_rank = 0
    cfg, _ = config_from_args(family, args, torch.bfloat16)
    name, layer_cfgs = model_name_and_layer_configs(family, cfg)
    engine = GalvatronSearchEngine(args)
    engine.set_search_engine_info(program_dir(family), layer_cfgs, name)
    engine.initialize_search_engine()
    if getattr(args, "check_cost_model", None):
        import json
        bsz, chunk, min_tp = (int(x) for x in args.check_cost_model.split(","))
        table = engine.check_cost_model(bsz, chunk, min_tp)
        tokens = bsz * cfg.seq_length
        for row in table:
            row["tokens_per_s"] = tokens / row["time_s"] if row["time_s"] > 0 else None
        print("COST_MODEL " + json.dumps({"bsz": bsz, "chunk": chunk, "min_tp": min_tp, "seq": cfg.seq_length, "rows": table}), flush=True)
        return table
    if getattr(args, "explain_plan", None):
        import json
        from ..utils.config_utils import read_json_config
        report = engine.explain_plan(read_json_config(args.explain_plan))
        report["tokens_per_s"] = report["throughput_samples_per_s"] * cfg.seq_length
        print("PLAN_REPORT " + json.dumps(report), flush=True)
        for st, (m, t) in enumerate(zip(report["stage_memory_mb"], report["stage_time_s"])):
            print("stage %d: %.0f MB, %.4f s" % (st, m, t))
        print("step %.4f s, %.1f samples/s" % (report["step_time_s"], report["throughput_samples_per_s"]))
        return report
    if getattr(args, "max_cp_deg", 1) > 1:
        from ..search.context_parallel import search_with_context_parallel
        for c, layer in zip(layer_cfgs, [cfg] * len(layer_cfgs)):
            c.setdefault("kv_hidden_size", cfg.hidden_size // cfg.num_heads * (cfg.num_kv_heads or cfg.num_heads))
        return search_with_context_parallel(args, program_dir(family), layer_cfgs, name, args.max_cp_deg)["throughput"]
    return engine.parallelism_optimization()
