"""Worker of the multi-process tests: trains a tiny model under a plan and prints the per-step losses.

Launched by tests through ``torch.distributed.run`` (gloo on CPU, nccl on GPUs); also runs single-process
(world size 1) to produce the un-parallelised baseline."""
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from hetu_galvatron_b200.core.hybrid_model import construct_hybrid_parallel_model  # noqa: E402
from hetu_galvatron_b200.core.plan import HybridPlan  # noqa: E402
from hetu_galvatron_b200.models import build_model_specs  # noqa: E402


def main():
    spec = json.loads(sys.argv[1])
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    use_cuda = spec.get("device", "cpu") == "cuda"
    if use_cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    else:
        device = torch.device("cpu")
    if world > 1:
        dist.init_process_group("nccl" if use_cuda else "gloo")
    dtype = {"fp32": torch.float32, "bf16": torch.bfloat16}[spec.get("dtype", "fp32")]
    cfg, specs = build_model_specs(spec["family"], dtype=dtype, **spec["model"])
    n_layers = len([s for s in specs if s.layer_index is not None])
    if "plan_json" in spec:
        plan = HybridPlan.from_json(spec["plan_json"], n_layers, sequence_parallel=spec.get("sequence_parallel", False))
    else:
        plan = HybridPlan.from_global(n_layers, world, **spec.get("plan", {}))
    import contextlib
    from hetu_galvatron_b200.models.transformer import deferred_init
    with (deferred_init() if spec.get("defer_init") else contextlib.nullcontext()):
        model = construct_hybrid_parallel_model(cfg, plan, specs, device, impl=spec.get("impl", "nccl"),
                                                async_grad_reduce=spec.get("async_grad_reduce", True))
    from hetu_galvatron_b200.models import synthetic_batch
    losses = []
    skipped = []
    from hetu_galvatron_b200.core.checkpoint import load_model, save_model
    start = 0
    if "load" in spec:
        load_model(model, spec["load"]["dir"], spec["family"], iteration=spec["load"].get("iter"),
                   allow_plan_change=spec["load"].get("allow_plan_change", False))
        start = spec["load"].get("start", spec["load"].get("iter") or 0)
    for it in range(start, spec.get("steps", 3)):
        batch = synthetic_batch(spec["family"], cfg, plan.global_bsz, seed=spec.get("seed", 100) + it, device=device,
                                **({"padded": True} if spec.get("padded") else {}))
        if spec.get("scramble_padding") and len(batch) > 2 and "attention_mask" in batch[2]:
            # other token ids at the padded positions: a working padding mask makes the loss independent of them
            ids = batch[0].clone()
            pad = batch[2]["attention_mask"] == 0
            ids[pad] = (ids[pad] + 7) % cfg.vocab_size
            extra = dict(batch[2])
            if "decoder_attention_mask" in extra:
                dec = extra["decoder_input_ids"].clone()
                dpad = extra["decoder_attention_mask"] == 0
                dec[dpad] = (dec[dpad] + 11) % cfg.vocab_size
                extra["decoder_input_ids"] = dec
            batch = (ids, batch[1], extra)
        lo, hi = model.batch_slice()
        batch = tuple(t[lo:hi] if torch.is_tensor(t) else {k: v[lo:hi] for k, v in t.items()} for t in batch)
        scale = float(spec.get("loss_scale", 1.0))
        if scale != 1.0:
            model.set_loss_scale(scale)
        loss = model.forward_backward(batch, it)
        if spec.get("poison") and spec["poison"]["iter"] == it and spec["poison"]["rank"] == rank:
            # what an fp16 overflow leaves behind, on ONE rank only: every rank has to skip the step all the same
            bucket = next(b for b in model.engine.buckets if b.numel and b.grad_shard is not None)
            bucket.grad_shard.view(-1)[0] = float("inf")
        model.optimizer_step(spec.get("lr", 1e-3), max_grad_norm=spec.get("clip", 1.0), loss_scale=scale)
        skipped.append(bool(model.engine.last_step_skipped))
        model.zero_grad()
        if "save" in spec and it + 1 == spec["save"]["iter"]:
            save_model(model, spec["save"]["dir"], spec["family"], it + 1, portable_optimizer=spec["save"].get("portable", False))
        loss = model.mean_loss_over_ranks(loss)
        if loss is not None:
            losses.append(float(loss))
    if spec.get("report_skipped"):
        flags = [None] * world
        if world > 1:
            dist.all_gather_object(flags, skipped)
        else:
            flags = [skipped]
        if rank == world - 1:
            print("SKIPPED " + json.dumps(flags), flush=True)
    if rank == world - 1:
        print("LOSSES " + json.dumps(losses), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
