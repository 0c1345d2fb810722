"""Headline benchmark: Llama-2-7B-shape training tokens/s (bf16, seq 4096, 8 sequences per GPU, synthetic
uniform tokens, random-init weights), timed on the device with CUDA events, max over ranks.

    python bench.py --gpus 1 --steps 4 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the unmodified reference from baseline/_ref, same metric/config

Every timed step is a full training step: forward + backward over all micro-batches, gradient reduction,
gradient-norm clipping and the AdamW update. Weak scaling: the per-GPU batch is fixed (global batch = 8 * N,
i.e. 64 sequences on 8 GPUs as in the baseline configuration).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL = "llama-7b"
SEQ = 4096
SEQS_PER_GPU = 8


class ClockSampler:
    """Samples SM clocks / throttle reasons of this process's GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax = float(parts[2])
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm)}


def run_ours(args) -> dict:
    import torch
    import torch.distributed as dist

    from hetu_galvatron_b200.core.hybrid_model import construct_hybrid_parallel_model
    from hetu_galvatron_b200.core.plan import HybridPlan
    from hetu_galvatron_b200.models.llama import llama_config, llama_specs
    from hetu_galvatron_b200.ops import _lib

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    n = world
    cfg = llama_config(args.model, seq_length=args.seq, dtype=torch.bfloat16)
    if args.layers:
        cfg.num_layers = args.layers
    global_bsz = args.seqs_per_gpu * n
    chunks = args.chunks or max(args.seqs_per_gpu // args.micro_batch, 1)
    if args.plan:
        plan = HybridPlan.from_json(args.plan, cfg.num_layers)
        plan.global_bsz, plan.chunks = global_bsz, chunks
        parallelism = "plan:" + os.path.basename(args.plan)
    else:
        plan = HybridPlan.from_global(cfg.num_layers, n, pp_deg=1, global_tp_deg=1, sdp=int(args.zero3),
                                      global_cp_deg=args.cp, vocab_cp=args.cp,
                                      global_checkpoint=int(args.checkpoint), chunks=chunks, global_bsz=global_bsz,
                                      default_dp_type="zero2" if n > 1 else "ddp")
        parallelism = ("dp%d-zero2" % (n // args.cp) if n > args.cp else "single") + ("-sdp" if args.zero3 else "") + \
            ("-cp%d" % args.cp if args.cp > 1 else "")
    # "auto": this package's peer-memory kernels for every collective of the step whenever there is more than one GPU
    # (gradient reduce-scatter, AdamW + parameter push, ZeRO-3 gathers, tensor/sequence-parallel GEMM+collective);
    # "nccl" keeps torch.distributed collectives (the library baseline of the same engine)
    want = args.comm_impl if args.comm_impl != "auto" else ("fused" if n > 1 else "nccl")
    def make_model(impl):
        return construct_hybrid_parallel_model(cfg, plan, llama_specs(cfg), device, impl=impl,
                                               grad_dtype=torch.float32 if args.fp32_grads else torch.bfloat16)

    def all_ranks_ok(ok: bool) -> bool:
        if world == 1:
            return ok
        flag = torch.tensor([int(ok)], dtype=torch.int32, device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        return bool(flag.item())

    def drop_model():
        import gc

        from hetu_galvatron_b200.parallel import symm
        gc.collect()
        torch.cuda.synchronize()
        symm.release_workspaces()
        torch.cuda.empty_cache()

    # The peer-memory engine needs symmetric allocations mapped by every rank of a group. Where they cannot be had (or
    # its kernels report an error in the first step, checked below) every rank falls back to the library collectives
    # together and the run says so under notes.comm_fallback; GV_BENCH_FAIL_FUSED=1 forces that path (a drill).
    comm_fallback = None
    model = None
    try:
        if want == "fused" and os.environ.get("GV_BENCH_FAIL_FUSED") == "1":
            raise RuntimeError("forced by GV_BENCH_FAIL_FUSED")
        model = make_model(want)
    except Exception as exc:
        if want != "fused":
            raise
        comm_fallback = "construction: %s: %s" % (type(exc).__name__, str(exc)[:200])
    if want == "fused" and not all_ranks_ok(comm_fallback is None):
        comm_fallback = comm_fallback or "construction failed on another rank"
        model = None
        drop_model()
        want = "nccl"
        model = make_model(want)
    # what was asked for; the data-parallel engine reports what it really runs on (plans without data parallelism have
    # no sharded bucket: there the label only covers the tensor / sequence / context-parallel paths)
    engine_impl = model.engine.comm_impl
    comm_impl = "none (single GPU)" if n == 1 else (want if engine_impl == want else "%s (zero engine: %s)" % (want, engine_impl))
    local_bsz = model.local_batch_size()
    # ranks that share a data-parallel slice (tensor/context-parallel peers) must be fed the same tokens
    g = torch.Generator().manual_seed(1234 + model.batch_slice()[0])
    # synthetic data in pinned host memory; one fresh batch per step is copied to the device inside the step
    n_host = args.warmup + 2 * args.steps + 2        # never revisit a batch: a 7B model memorises a repeated one at once
    host_tokens = [torch.randint(0, cfg.vocab_size, (local_bsz, args.seq + 1), generator=g).pin_memory() for _ in range(min(n_host, 64))]
    peak_lr, lr_warmup_steps = 1e-4, 50
    counter = {"step": 0}

    def step(i: int, e2e: bool):
        k = counter["step"]                # a different batch every step of the run, linear learning-rate warm-up
        counter["step"] = k + 1
        lr = peak_lr * min(1.0, (k + 1) / lr_warmup_steps)
        if e2e:
            tok = host_tokens[k % len(host_tokens)].to(device, non_blocking=True)
        else:
            tok = dev_tokens[k % len(dev_tokens)]
        loss = model.forward_backward((tok[:, :-1], tok[:, 1:]), i)
        model.optimizer_step(lr, beta1=0.9, beta2=0.95, weight_decay=0.1, max_grad_norm=1.0)
        model.zero_grad()
        if e2e:
            # device -> host read of the step's result (the loss lives on the last pipeline stage; other stages
            # read back their gradient norm, the scalar their step produced)
            return float(loss.item()) if loss is not None else float(model.engine.last_norm.item())
        return loss

    dev_tokens = [t.to(device) for t in host_tokens]

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(e2e: bool, steps: int):
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        last = None
        for i in range(steps):
            last = step(i, e2e)
        e1.record()
        sync()
        ms = e0.elapsed_time(e1)
        t = torch.tensor([ms], device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), last

    for i in range(args.warmup):
        step(i, False)
        if i == 0 and want == "fused":
            # the first step has exercised every kernel of the engine: a bounded wait that ran out shows in the error word
            torch.cuda.synchronize()
            first_err = _lib.read_error()
            if not all_ranks_ok(first_err is None):
                comm_fallback = "first step: kernel error %s" % (first_err,)
                model = None
                drop_model()
                want = "nccl"
                model = make_model(want)
                comm_impl = "nccl"
    sync()
    if args.gaps:
        # one steady step under the CUDA activity tracer: how much of the step's span has no kernel running
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            step(0, False)
            torch.cuda.synchronize()
        ev = sorted(((e.time_range.start, e.time_range.end, e.name) for e in prof.events()
                     if e.device_type == torch.autograd.DeviceType.CUDA and e.time_range.end > e.time_range.start), key=lambda t: t[0])
        busy, gaps, cur_end = 0.0, [], ev[0][0]
        for st, en, name in ev:
            if st > cur_end:
                gaps.append((st - cur_end, name))
                busy += en - st
                cur_end = en
            elif en > cur_end:
                busy += en - cur_end
                cur_end = en
        span = cur_end - ev[0][0]
        gaps.sort(reverse=True)
        # whose kernels: this package's (namespace gv), communication library, everything else (torch / cuBLAS / memset)
        other = {}
        own = nccl = 0
        own_us = other_us = 0.0
        for st, en, name in ev:
            if "gv::" in name:
                own += 1
                own_us += en - st
            elif name.startswith("nccl"):
                nccl += 1
            else:
                c = other.setdefault(name[:70], [0, 0.0])
                c[0] += 1
                c[1] += en - st
                other_us += en - st
        top_other = sorted(other.items(), key=lambda kv: -kv[1][0])[:10]
        if rank == 0:
            print(json.dumps({"gaps": {"kernels": len(ev), "span_ms": span / 1e3, "busy_ms": busy / 1e3, "idle_ms": (span - busy) / 1e3,
                                       "idle_fraction": (span - busy) / span, "gaps_over_50us": sum(1 for g in gaps if g[0] > 50),
                                       "largest_gaps_us": [(round(g[0], 1), g[1][:60]) for g in gaps[:8]],
                                       "own_kernels": own, "own_kernel_ms": own_us / 1e3, "nccl_kernels": nccl,
                                       "other_kernels": len(ev) - own - nccl, "other_kernel_ms": other_us / 1e3,
                                       "top_other_kernels": [(k, v[0], round(v[1] / 1e3, 3)) for k, v in top_other]}}), flush=True)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = _lib.launch_count()
    ms_total, _ = timed(False, args.steps)
    launches = _lib.launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else {}
    ms_e2e, last_loss = timed(True, args.steps)
    err = _lib.read_error()
    tokens = global_bsz * args.seq
    ms_per_step = ms_total / args.steps
    value = tokens / (ms_per_step / 1e3)
    e2e_value = tokens / (ms_e2e / args.steps / 1e3)
    mem_gb = torch.cuda.max_memory_allocated() / 2 ** 30
    # peer-mapped (symmetric) allocations are made outside torch's caching allocator: the buckets of the fused data-parallel
    # engine and the cached per-shape workspaces of the fused tensor-parallel paths
    symm_gb = 0.0
    try:
        from hetu_galvatron_b200.parallel import symm as _symm
        symm_bytes = _symm.workspace_stats()["bytes"]
        for b in model.engine.buckets:
            f = getattr(b, "fused", None)
            if f is not None:
                symm_bytes += f.ws.nbytes
        symm_gb = symm_bytes / 2 ** 30
    except Exception:
        pass
    out = {
        "metric": "%s_train_tokens_per_s" % args.model.replace("-", "").replace(".", "_"), "value": value, "unit": "tokens/s", "n_gpus": n, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform token ids, random-init weights",
        "config": {"model": ("llama-2-7b-shape (32L h4096 32 heads ffn11008 vocab32000)" if args.model == MODEL else args.model) if not args.layers else "%s-shape %d layers" % (args.model, args.layers),
                   "global_batch": global_bsz, "seq_len": args.seq, "micro_batch": args.micro_batch,
                   "parallelism": parallelism, "checkpoint": int(args.checkpoint)},
        "notes": {"l2": "inputs larger than L2 (13.5 GB of bf16 weights streamed per micro-batch)",
                  "grads": "fp32" if args.fp32_grads else "bf16", "comm_impl": comm_impl,
                  "optimizer": "AdamW betas 0.9/0.95 eps 1e-8 decay 0.1, clip 1.0, linear warm-up"},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": local_bsz * (args.seq + 1) * 8,
                "d2h_bytes_per_step": 4, "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": launches,
        "peak_mem_gb": mem_gb, "symmetric_mem_gb": symm_gb, "last_loss": last_loss, "kernel_error": err, "impl": "ours",
    }
    if comm_fallback is not None:
        out["notes"]["comm_fallback"] = comm_fallback
    if world > 1:
        dist.destroy_process_group()
    return out if rank == 0 else {}


def run_reference(args) -> dict:
    from baseline.run_ref import run_reference_bench

    return run_reference_bench(args)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default=MODEL, help="llama-family size from models/meta_configs (the headline metric is llama-7b)")
    ap.add_argument("--seq", type=int, default=SEQ)
    ap.add_argument("--seqs-per-gpu", type=int, default=SEQS_PER_GPU)
    ap.add_argument("--micro-batch", type=int, default=2)
    ap.add_argument("--layers", type=int, default=0, help="debug only: fewer layers (result is then not the headline metric)")
    ap.add_argument("--zero3", action="store_true")
    ap.add_argument("--checkpoint", action="store_true")
    ap.add_argument("--fp32-grads", action="store_true")
    ap.add_argument("--chunks", type=int, default=0, help="micro-batches per step (default: seqs-per-gpu / micro-batch)")
    ap.add_argument("--gaps", action="store_true", help="also trace one step and report the time no kernel was running")
    ap.add_argument("--cp", type=int, default=1, help="context-parallel degree (zigzag ring attention) of the default plan")
    ap.add_argument("--plan", default=None, help="strategy JSON to run instead of the default data-parallel plan")
    ap.add_argument("--comm-impl", default="auto", choices=["auto", "nccl", "fused"],
                    help="auto = fused (own peer-memory kernels) when more than one GPU runs, nccl = torch.distributed collectives")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus != world and args.gpus > 1 and "RANK" not in os.environ:
        # convenience: re-launch under torchrun
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(args.gpus),
               "--master-addr", "127.0.0.1", "--master-port", "29531", os.path.abspath(__file__)] + sys.argv[1:]
        sys.exit(subprocess.call(cmd))
    out = run_reference(args) if args.impl == "reference" else run_ours(args)
    if out:
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
