"""Worker for tests/test_fused_gpu.py: each fused compute + collective op against its library-collective version."""
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from hetu_galvatron_b200.ops import _lib  # noqa: E402
from hetu_galvatron_b200.ops.gemm import gemm  # noqa: E402
from hetu_galvatron_b200.parallel import collectives as C  # noqa: E402
from hetu_galvatron_b200.parallel import fused  # noqa: E402
from hetu_galvatron_b200.parallel.mesh import Mesh  # noqa: E402
from hetu_galvatron_b200.parallel.reshard import Layout, _redistribute_nccl  # noqa: E402
from hetu_galvatron_b200.parallel.symm import workspace  # noqa: E402
from hetu_galvatron_b200.parallel.ulysses import _ColsToRanks, _RowsToRanks, _send_columns  # noqa: E402


def rel(a, b):
    return ((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-6)).item()


def main():
    spec = json.loads(sys.argv[1]) if len(sys.argv) > 1 else {}
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl")
    mesh = Mesh(world, rank, 1)
    cg = mesh.group("tp", world)
    pg = cg.group
    torch.manual_seed(100 + rank)
    res = {}
    rows, h, f = spec.get("rows", 512), spec.get("hidden", 1024), spec.get("ffn", 2048)
    for rep in range(3):          # three rounds: both workspace parities get reused
        x = torch.randn(rows, h, device=dev, dtype=torch.bfloat16)
        torch.manual_seed(7)
        Wc = (torch.randn(f // world, h, device=dev) * 0.05).bfloat16()      # column-parallel shard
        Wr = (torch.randn(h, f // world, device=dev) * 0.05).bfloat16()      # row-parallel shard
        torch.manual_seed(100 + rank + rep)
        # F1: all-gather -> GEMM
        ref = gemm(C.all_gather_first_dim(x, pg), Wc)
        res["ag_gemm"] = max(res.get("ag_gemm", 0), rel(fused.allgather_gemm(x, Wc, pg), ref))
        # F2: GEMM -> reduce-scatter (+ residual)
        a = torch.randn(rows * world, f // world, device=dev, dtype=torch.bfloat16)
        r = torch.randn(rows, h, device=dev, dtype=torch.bfloat16)
        ref = C.reduce_scatter_first_dim(gemm(a, Wr, out_dtype=torch.float32), pg) + r.float()
        res["gemm_rs"] = max(res.get("gemm_rs", 0), rel(fused.gemm_reduce(a, Wr, pg, scatter=True, residual=r), ref))
        # F2b: input-gradient GEMM -> reduce-scatter (weight used as stored)
        dy = torch.randn(rows * world, f // world, device=dev, dtype=torch.bfloat16)
        ref = C.reduce_scatter_first_dim(gemm(dy, Wc, b_mn=True, out_dtype=torch.float32), pg)
        res["dgrad_rs"] = max(res.get("dgrad_rs", 0), rel(fused.gemm_reduce(dy, Wc, pg, scatter=True, b_mn=True), ref))
        # F3: GEMM -> all-reduce
        ref = C.all_reduce_(gemm(a, Wr, out_dtype=torch.float32), pg)
        res["gemm_ar"] = max(res.get("gemm_ar", 0), rel(fused.gemm_reduce(a, Wr, pg, scatter=False), ref))
        # pull all-gather
        shard = torch.randn(4096 + 8 * rep, device=dev, dtype=torch.bfloat16)
        ref = C.all_gather_first_dim(shard, pg)
        res["ag_pull"] = max(res.get("ag_pull", 0), rel(fused.allgather_pull(shard, cg, "t"), ref))
        # U1 / U2: Ulysses projections fused with the exchanges
        hq, hk, dh = 8, 8, 128
        idx = _send_columns(hq, hk, dh, world, dev)
        torch.manual_seed(11)
        Wqkv = (torch.randn((hq + 2 * hk) * dh, h, device=dev) * 0.05).bfloat16()
        Wo = (torch.randn(h, hq * dh, device=dev) * 0.05).bfloat16()
        torch.manual_seed(100 + rank + rep)
        ref = _ColsToRanks.apply(gemm(x, Wqkv), idx, pg)
        got = fused.qkv_to_heads(x, Wqkv, None, idx, cg)
        res["u1"] = max(res.get("u1", 0), rel(got, ref))
        o = torch.randn(rows * world, hq // world * dh, device=dev, dtype=torch.bfloat16)
        ref = gemm(_RowsToRanks.apply(o, world, pg), Wo, out_dtype=torch.float32) + r.float()
        res["u2"] = max(res.get("u2", 0), rel(fused.heads_to_out(o, Wo, None, r, cg), ref))
        # R1: reshard between layouts
        B, seq = 4, 64
        for old, new in ((Layout(1, 1, False), Layout(world, 1, True)), (Layout(world, 1, True), Layout(1, 1, False)),
                         (Layout(world, 1, False), Layout(1, 1, False))):
            s_old = seq // old.seq_parts()
            b_old = B // old.dp(world)
            torch.manual_seed(5)
            full = torch.randn(seq, B, 256, device=dev, dtype=torch.bfloat16)
            from hetu_galvatron_b200.parallel.reshard import batch_range, seq_positions
            pos = seq_positions(old, rank, seq).to(dev)
            lo, hi = batch_range(old, rank, world, B)
            piece = full[pos][:, lo:hi].contiguous()
            ref = _redistribute_nccl(piece, old, new, mesh, B, seq)
            got = fused.reshard(piece, old, new, mesh, B, seq)
            res["reshard"] = max(res.get("reshard", 0), rel(got, ref))
        # plain NVLink collectives: pull p2p, all-to-all, two-shot all-reduce (peer loads; in-switch when offered)
        buf = torch.randn(world * 4096, device=dev, dtype=torch.bfloat16)
        ref = C.all_gather_first_dim(buf, pg).view(world, -1)[(rank + 1) % world]
        res["p2p"] = max(res.get("p2p", 0), rel(fused.p2p_pull(buf, (rank + 1) % world, cg), ref))
        ref = torch.empty_like(buf)
        dist.all_to_all_single(ref, buf, group=pg)
        res["a2a"] = max(res.get("a2a", 0), rel(fused.alltoall_pull(buf, cg), ref))
        ref = C.all_reduce_(buf.float(), pg)
        res["allreduce"] = max(res.get("allreduce", 0), rel(fused.allreduce_symm(buf, cg), ref))
        if spec.get("multimem"):
            res["allreduce_mm"] = max(res.get("allreduce_mm", 0), rel(fused.allreduce_symm(buf, cg, tag="mm", multimem=True), ref))
        # Z2: gradient reduce-scatter + AdamW + parameter push in one kernel vs reduce-scatter + torch AdamW
        n = world * 4096
        torch.manual_seed(50 + rank + rep)
        grad = torch.randn(n, device=dev, dtype=torch.bfloat16)
        torch.manual_seed(3)
        full_master = torch.randn(n, device=dev)
        sh = n // world
        master = full_master[rank * sh:(rank + 1) * sh].clone()
        m1, v1 = torch.zeros(sh, device=dev), torch.zeros(sh, device=dev)
        got = fused.rs_adamw(grad, master, m1, v1, cg, step=1, lr=1e-2, beta1=0.9, beta2=0.95, weight_decay=0.1,
                             grad_scale=1.0 / world).float()
        gsum = C.all_reduce_(grad.float(), pg) / world
        mm = 0.1 * gsum
        vv = 0.05 * gsum * gsum
        ref = full_master - 1e-2 * ((mm / 0.1) / ((vv / 0.05).sqrt() + 1e-8) + 0.1 * full_master)
        res["rs_adamw"] = max(res.get("rs_adamw", 0), rel(got, ref.bfloat16().float()))
    torch.cuda.synchronize()
    # bounded wait: nothing ever announces epoch 12345 on slot 14; the kernel must give up and report it
    ws = workspace(cg, 4096, tag="timeout_probe")
    ws.wait(14, (rank + 1) % world, 12345, timeout_ms=200)
    torch.cuda.synchronize()
    err = _lib.read_error()
    res["timeout_reported"] = bool(err and err["site"] == 0x32)
    res["stale_error"] = _lib.read_error() is not None
    dist.barrier()
    if rank == world - 1:
        print("LOSSES " + json.dumps(res), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
