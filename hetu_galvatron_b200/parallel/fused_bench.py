"""Micro-benchmark of the fused compute + collective kernels against their library-collective sequences.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29533 \
        -m hetu_galvatron_b200.parallel.fused_bench --out fused_bench.json

Shapes are the tensor-parallel linears of a Llama-7B layer (hidden 4096, ffn 11008) on ``--tokens`` tokens per
micro-batch. Every number is timed with CUDA events on the launching stream after warm-up, inputs rotate through
buffers that together exceed L2, and the reported time is the maximum over ranks. The roofline time of a fused op is
the slower of FLOPs / measured GEMM peak and bytes-over-NVLink / measured peer bandwidth.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..ops.gemm import gemm
from . import collectives as C
from . import fused
from .mesh import Mesh


def _time(fn, iters: int, warmup: int = 3) -> float:
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=11008)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--peak-tflops", type=float, default=0.0, help="measured cuBLAS bf16 peak; 0 = read MEASURED_PEAKS.json")
    ap.add_argument("--link-gbs", type=float, default=770.0)
    ap.add_argument("--out", default=None)
    a = ap.parse_args(argv)
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl")
    peak = a.peak_tflops
    if not peak:
        try:
            here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
            peak = float(json.load(open(os.path.join(here, "MEASURED_PEAKS.json")))["bf16_tflops"])
        except Exception:
            peak = 1590.0
    mesh = Mesh(world, rank, 1)
    cg = mesh.group("tp", world)
    pg = cg.group
    T, h, f = a.tokens, a.hidden, a.ffn
    rows = T // world
    NB = 3   # rotating buffers
    xs = [torch.randn(rows, h, device=dev, dtype=torch.bfloat16) for _ in range(NB)]
    w_up = [(torch.randn(2 * f // world, h, device=dev) * 0.02).bfloat16() for _ in range(NB)]
    w_qkv = [(torch.randn(3 * h // world, h, device=dev) * 0.02).bfloat16() for _ in range(NB)]
    acts = [torch.randn(T, f // world, device=dev, dtype=torch.bfloat16) for _ in range(NB)]
    w_down = [(torch.randn(h, f // world, device=dev) * 0.02).bfloat16() for _ in range(NB)]
    attn = [torch.randn(T, h // world, device=dev, dtype=torch.bfloat16) for _ in range(NB)]
    w_o = [(torch.randn(h, h // world, device=dev) * 0.02).bfloat16() for _ in range(NB)]
    res = [torch.randn(rows, h, device=dev, dtype=torch.bfloat16) for _ in range(NB)]
    results = {}

    def record(name, flops, link_bytes, t_lib, t_fused, t_gemm):
        roof = max(flops / (peak * 1e12), link_bytes / (a.link_gbs * 1e9)) * 1e3
        results[name] = {"library_ms": round(t_lib, 4), "fused_ms": round(t_fused, 4), "gemm_only_ms": round(t_gemm, 4),
                         "speedup": round(t_lib / t_fused, 3), "roofline_ms": round(roof, 4),
                         "fused_frac_of_roofline": round(roof / t_fused, 3),
                         "tflops_fused": round(flops / t_fused / 1e9, 1)}

    # all-gather -> GEMM (QKV and gate|up projections under sequence parallelism)
    for name, ws in (("ag_gemm_qkv", w_qkv), ("ag_gemm_up", w_up)):
        n = ws[0].shape[0]
        t_lib = _time(lambda i: gemm(C.all_gather_first_dim(xs[i % NB], pg), ws[i % NB]), a.iters)
        t_fus = _time(lambda i: fused.allgather_gemm(xs[i % NB], ws[i % NB], pg), a.iters)
        full = torch.randn(T, h, device=dev, dtype=torch.bfloat16)
        t_g = _time(lambda i: gemm(full, ws[i % NB]), a.iters)
        record(name, 2.0 * T * n * h, (world - 1) * rows * h * 2, t_lib, t_fus, t_g)
        del full
    # GEMM -> reduce-scatter (+ residual) (down and output projections)
    for name, xa, ws in (("gemm_rs_down", acts, w_down), ("gemm_rs_out", attn, w_o)):
        k = ws[0].shape[1]
        t_lib = _time(lambda i: C.reduce_scatter_first_dim(gemm(xa[i % NB], ws[i % NB]), pg).add_(res[i % NB]), a.iters)
        t_fus = _time(lambda i: fused.gemm_reduce(xa[i % NB], ws[i % NB], pg, scatter=True, residual=res[i % NB]), a.iters)
        t_g = _time(lambda i: gemm(xa[i % NB], ws[i % NB]), a.iters)
        record(name, 2.0 * T * h * k, (world - 1) * rows * h * 2, t_lib, t_fus, t_g)
    # GEMM -> all-reduce (tensor parallelism without sequence parallelism)
    t_lib = _time(lambda i: C.all_reduce_(gemm(acts[i % NB], w_down[i % NB]), pg), a.iters)
    t_fus = _time(lambda i: fused.gemm_reduce(acts[i % NB], w_down[i % NB], pg, scatter=False), a.iters)
    t_g = _time(lambda i: gemm(acts[i % NB], w_down[i % NB]), a.iters)
    record("gemm_ar_down", 2.0 * T * h * (f // world), 2 * (world - 1) * rows * h * 2, t_lib, t_fus, t_g)
    # pull all-gather vs NCCL all-gather (ZeRO-3 parameter gather of one 7B layer: 202 M bf16 / world)
    shard = torch.randn(202_383_360 // world // 8 * 8, device=dev, dtype=torch.bfloat16)
    out = torch.empty(world * shard.numel(), device=dev, dtype=torch.bfloat16)
    t_lib = _time(lambda i: dist.all_gather_into_tensor(out, shard, group=pg), a.iters)
    t_fus = _time(lambda i: fused.allgather_pull(shard, cg, "bench", out=out), a.iters)
    link = (world - 1) * shard.numel() * 2
    results["allgather_params"] = {"library_ms": round(t_lib, 4), "fused_ms": round(t_fus, 4), "speedup": round(t_lib / t_fus, 3),
                                   "fused_GBps_in": round(link / t_fus / 1e6, 1), "library_GBps_in": round(link / t_lib / 1e6, 1),
                                   "fused_frac_of_link": round(link / t_fus / 1e6 / a.link_gbs, 3)}
    from ..ops import _lib
    results["_meta"] = {"world": world, "tokens": T, "hidden": h, "ffn": f, "peak_tflops_measured": peak,
                        "link_gbs_measured": a.link_gbs, "kernel_error": _lib.read_error(),
                        "nvls": os.environ.get("NCCL_NVLS_ENABLE", "default")}
    if rank == 0:
        print("FUSED_BENCH " + json.dumps(results), flush=True)
        if a.out:
            json.dump(results, open(a.out, "w"), indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
