"""Reference arm of bench.py: the unmodified reference (installed under ``baseline/_ref``) trained through its own
public API -- ``initialize_galvatron`` -> ``llama_model_hp`` -> ``GalvatronModel.forward_backward`` + the optimizer
its ``train_dist_random.py`` uses -- on the same metric and configuration as the main arm (Llama-2-7B shape, bf16,
seq 4096, 8 sequences per GPU, synthetic tokens, random init). None of this package's models, kernels or engine
is imported on this path. Third-party native packages that the image lacks (apex, amp_C, flash-attn's rms_norm
op) are replaced by the PyTorch stand-ins of ``baseline/shims/ref_shims.py``.
"""
from __future__ import annotations

import json
import os
import sys
import traceback

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")


def _flags(args, world: int, micro_batch: int, checkpoint: int, sdp: int) -> list:
    chunks = max(args.seqs_per_gpu // micro_batch, 1)
    return [
        "--model_size", "llama-7b", "--set_model_config_manually", "0", "--set_layernum_manually", "0" if not args.layers else "1",
        "--set_seqlen_manually", "1", "--vocab_size", "32000", "--hidden_size", "4096",
        "--num_hidden_layers", str(args.layers or 32), "--num_attention_heads", "32", "--seq_length", str(args.seq),
        "--global_train_batch_size", str(args.seqs_per_gpu * world), "--train-iters", "10000",
        # optimizer and schedule flags as the reference's scripts/train_dist.sh passes them, with the betas / eps /
        # decay of the main arm (AdamW 0.9 / 0.95, eps 1e-8, decay 0.1, warm-up then cosine decay)
        "--lr", "1e-4", "--min-lr", "1e-5", "--lr-decay-style", "cosine", "--lr-warmup-fraction", "0.005",
        "--weight-decay", "0.1", "--adam_weight_decay", "0.1", "--adam-beta1", "0.9", "--adam-beta2", "0.95",
        "--adam-eps", "1e-8", "--dropout_prob", "0.0", "--check_loss", "0", "--profile", "0",
        "--pp_deg", "1", "--global_tp_deg", "1", "--global_tp_consec", "1", "--sdp", str(sdp),
        "--global_checkpoint", str(checkpoint), "--vocab_tp", "1", "--chunks", str(chunks),
        "--pipeline_type", "pipedream_flush", "--default_dp_type", "zero2", "--mixed_precision", "bf16",
        "--use-flash-attn", "--initialize_on_meta", "1", "--clip-grad", "1.0",
    ]


def _run(args, micro_batch: int, checkpoint: int, sdp: int) -> dict:
    import torch

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29577")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("LOCAL_RANK", "0")
    world = int(os.environ["WORLD_SIZE"])
    rank = int(os.environ["RANK"])
    local_rank = int(os.environ["LOCAL_RANK"])
    sys.path.insert(0, os.path.join(HERE, "shims"))
    sys.path.insert(0, REF_DIR)
    import ref_shims

    ref_shims.install()
    saved_argv = sys.argv
    sys.argv = [os.path.join(REF_DIR, "galvatron", "models", "llama_hf", "train_dist_random.py"), "--local-rank", str(local_rank)] \
        + _flags(args, world, micro_batch, checkpoint, sdp)
    try:
        from galvatron.core import initialize_galvatron
        from galvatron.core.runtime.utils import clip_grad_norm
        from galvatron.models.llama_hf.arguments import model_args
        from galvatron.models.llama_hf.LlamaModel_hybrid_parallel import get_llama_config, get_runtime_profiler, llama_model_hp
        from galvatron.utils import set_seed

        a = initialize_galvatron(model_args, mode="train_dist")
        set_seed()
    finally:
        sys.argv = saved_argv
    import torch.distributed as dist

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    config = get_llama_config(a)
    model = llama_model_hp(config, a)
    # The reference's trainer (models/llama_hf/train_dist.py) builds its optimizer with
    # get_optimizer_and_param_scheduler: apex FusedAdam (here the fused torch AdamW stand-in) + Megatron's scheduler.
    # Should that factory fail on this image, fall back to what its train_dist_random.py does (torch Adam).
    opt_param_scheduler, optimizer_kind = None, "get_optimizer_and_param_scheduler (FusedAdam stand-in: torch AdamW fused)"
    try:
        from galvatron.core.runtime.utils import get_optimizer_and_param_scheduler

        a.distributed_checkpoint = getattr(a, "distributed_checkpoint", False)
        optimizer, opt_param_scheduler = get_optimizer_and_param_scheduler(model, a)
    except Exception as exc:
        if rank == 0:
            print("reference optimizer factory failed (%s: %s); using torch.optim.Adam as train_dist_random.py does"
                  % (type(exc).__name__, exc), file=sys.stderr)
        optimizer = torch.optim.Adam(model.parameters(), lr=a.lr, weight_decay=a.adam_weight_decay)
        optimizer_kind = "torch.optim.Adam (train_dist_random.py)"
    profiler = get_runtime_profiler(a, os.path.join(REF_DIR, "galvatron", "models", "llama_hf"), config)
    local_bsz = a.global_train_batch_size // world
    g = torch.Generator().manual_seed(1234 + rank)
    host = [torch.randint(0, 32000, (local_bsz, args.seq + 1), generator=g).pin_memory() for _ in range(4)]
    dev = [t.to(device) for t in host]

    def step(i, e2e):
        tok = host[i % 4].to(device, non_blocking=True) if e2e else dev[i % 4]
        batch = [tok[:, :-1].contiguous()]
        kwargs = {"attention_mask": None, "labels": tok[:, 1:].contiguous()}
        loss = model.forward_backward(batch, i, profiler, loss_func=None, **kwargs)
        clip_grad_norm(model, a.clip_grad)
        optimizer.step()
        if opt_param_scheduler is not None:
            opt_param_scheduler.step(increment=getattr(a, "global_batch_size", None) or a.global_train_batch_size)
        optimizer.zero_grad()
        if e2e and loss is not None:
            return float(loss.item() if hasattr(loss, "item") else loss)
        return loss

    def sync():
        dist.barrier()
        torch.cuda.synchronize()

    def timed(e2e, steps):
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        last = None
        for i in range(steps):
            last = step(i, e2e)
        e1.record()
        sync()
        t = torch.tensor([e0.elapsed_time(e1)], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), last

    for i in range(args.warmup):
        step(i, False)
    from bench import ClockSampler

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms, _ = timed(False, args.steps)
    clocks = sampler.stop() if rank == 0 else {}
    ms_e2e, last = timed(True, args.steps)
    tokens = a.global_train_batch_size * args.seq
    out = {
        "impl": "reference", "metric": "llama7b_train_tokens_per_s", "value": tokens / (ms / args.steps / 1e3), "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform token ids, random-init weights",
        "config": {"model": "llama-2-7b-shape (32L h4096 32 heads ffn11008 vocab32000)" if not args.layers else "llama-7b-shape %d layers" % args.layers,
                   "global_batch": a.global_train_batch_size, "seq_len": args.seq, "micro_batch": micro_batch,
                   "parallelism": ("dp%d-zero2" % world if world > 1 else "single") + ("-sdp" if sdp else ""),
                   "checkpoint": checkpoint},
        "notes": {"stack": "reference runtime: HF Llama skeleton + Megatron TP layers + FSDP1 + FlashAttention-2",
                  "optimizer": optimizer_kind,
                  "shims": "apex.FusedAdam->torch AdamW(fused), amp_C->torch._foreach, flash_attn.ops.rms_norm->torch rms_norm",
                  "memory": "at 1 GPU the unsharded fp32 optimizer state puts this arm near the device's memory limit; "
                            "its 1-GPU figure is allocator-bound"},
        "clocks": clocks,
        "e2e": {"value": tokens / (ms_e2e / args.steps / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": local_bsz * (args.seq + 1) * 8,
                "d2h_bytes_per_step": 4, "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": 0, "peak_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30, "last_loss": last,
    }
    return out if rank == 0 else {}


def run_reference_bench(args) -> dict:
    if not os.path.isdir(os.path.join(REF_DIR, "galvatron")):
        return {"impl": "reference", "unavailable": "reference is not installed under baseline/_ref"}
    attempts = [(args.micro_batch, int(args.checkpoint), int(args.zero3))]
    rank = int(os.environ.get("RANK", "0"))
    try:
        return _run(args, *attempts[0])
    except Exception as exc:  # one line, exit 0: the driver records the arm as unavailable
        msg = "%s: %s" % (type(exc).__name__, str(exc).replace("\n", " ")[:300])
        if rank == 0:
            traceback.print_exc(file=sys.stderr)
            return {"impl": "reference", "unavailable": msg}
        return {}
