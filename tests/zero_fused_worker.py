"""Worker of tests/test_zero_fused_gpu.py: inside ONE multi-GPU launch, trains the same tiny model under every
data-parallel flavour twice -- gradient / parameter traffic through torch.distributed (NCCL) and through this
package's peer-memory kernels -- and compares losses and final parameters. Prints one RESULT line."""
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from hetu_galvatron_b200.core.hybrid_model import construct_hybrid_parallel_model  # noqa: E402
from hetu_galvatron_b200.core.plan import HybridPlan  # noqa: E402
from hetu_galvatron_b200.models import build_model_specs, synthetic_batch  # noqa: E402
from hetu_galvatron_b200.ops import _lib  # noqa: E402


def train(spec, case, impl, device, world, profile_step=None):
    cfg, specs = build_model_specs("llama", dtype=torch.bfloat16, **spec["model"])
    n_layers = len([s for s in specs if s.layer_index is not None])
    plan = HybridPlan.from_global(n_layers, world, global_bsz=spec["global_bsz"], chunks=case["chunks"], sdp=int(case["dp"] == "zero3"),
                                  default_dp_type="ddp" if case["dp"] == "ddp" else "zero2",
                                  global_checkpoint=int(case.get("ckpt", 0)))
    model = construct_hybrid_parallel_model(cfg, plan, specs, device, impl=impl, async_grad_reduce=case["async"],
                                            grad_dtype=torch.bfloat16 if case.get("bf16_grads") else torch.float32)
    losses, kernels = [], []
    for it in range(spec["steps"]):
        batch = synthetic_batch("llama", cfg, plan.global_bsz, seed=100 + it, device=device)
        lo, hi = model.batch_slice()
        batch = tuple(t[lo:hi] for t in batch)

        def one_step():
            loss = model.forward_backward(batch, it)
            model.optimizer_step(1e-3, beta2=0.95, weight_decay=0.1, max_grad_norm=case["clip"])
            model.zero_grad()
            return loss

        if profile_step is not None and it == profile_step:
            from torch.profiler import ProfilerActivity, profile
            with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
                loss = one_step()
                torch.cuda.synchronize()
            kernels = sorted({e.name for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA})
        else:
            loss = one_step()
        losses.append(float(model.mean_loss_over_ranks(loss)))
    # checksum of the final parameters of every bucket (gathered where sharded)
    sums = []
    for b in model.engine.buckets:
        if b.numel:
            full = b.full_params()
            sums.append(float(sum(v.float().abs().sum() for v in full.values())))
    torch.cuda.synchronize()
    used = model.engine.comm_impl
    del model
    return losses, sums, used, kernels


def main():
    spec = json.loads(sys.argv[1])
    world = int(os.environ["WORLD_SIZE"])
    rank = int(os.environ["RANK"])
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    results = []
    for i, case in enumerate(spec["cases"]):
        ref_l, ref_s, used_ref, _ = train(spec, case, "nccl", device, world)
        got_l, got_s, used, kernels = train(spec, case, "fused", device, world, profile_step=2 if i == spec.get("profile_case", -1) else None)
        err = _lib.read_error()
        dl = max(abs(a - b) for a, b in zip(ref_l, got_l))
        ds = max(abs(a - b) / max(abs(a), 1.0) for a, b in zip(ref_s, got_s))
        results.append({"case": case, "loss_diff": dl, "param_rel_diff": ds, "impl_ref": used_ref, "impl": used, "kernel_error": err,
                        "losses": got_l, "ref_losses": ref_l,
                        "nccl_kernels": [k for k in kernels if "nccl" in k.lower()],
                        "own_comm_kernels": [k for k in kernels if any(t in k for t in ("grad_reduce", "adamw_push", "allgather_pull", "wait_zero", "wait_peers"))]})
    if rank == 0:
        print("RESULT " + json.dumps(results), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
