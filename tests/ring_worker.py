"""Worker of tests/test_ring_attention_cpu.py: zigzag ring attention over cp ranks against attention over the whole
sequence computed in-process (forward output and the gradients of q, k, v)."""
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from hetu_galvatron_b200.ops import functional as Fn  # noqa: E402
from hetu_galvatron_b200.parallel.mesh import Mesh  # noqa: E402
from hetu_galvatron_b200.parallel.ring_attention import ZigzagRingAttention  # noqa: E402


def zigzag_rows(cp, r, chunk):
    return list(range(r * chunk, (r + 1) * chunk)) + list(range((2 * cp - 1 - r) * chunk, (2 * cp - r) * chunk))


def main():
    spec = json.loads(sys.argv[1])
    use_cuda = spec.get("device") == "cuda"
    if use_cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dist.init_process_group("nccl" if use_cuda else "gloo")
    rank, cp = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu")
    dtype = torch.bfloat16 if use_cuda else torch.float32
    mesh = Mesh(cp, rank, 1)
    cg = mesh.group("cp", 1, cp)
    worst = 0.0
    for case in spec["cases"]:
        s, b, hq, hk, dh, causal = case["s"], case["b"], case["hq"], case["hk"], case["dh"], case["causal"]
        g = torch.Generator().manual_seed(7)
        q = torch.randn(s, b, hq, dh, generator=g).to(dev, dtype)
        k = torch.randn(s, b, hk, dh, generator=g).to(dev, dtype)
        v = torch.randn(s, b, hk, dh, generator=g).to(dev, dtype)
        do = torch.randn(s, b, hq, dh, generator=g).to(dev, dtype)
        scale = dh ** -0.5
        # whole-sequence reference
        qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
        o_ref, _ = Fn.attention_reference(qf.transpose(0, 1), kf.transpose(0, 1), vf.transpose(0, 1), causal, scale)
        o_ref = o_ref.transpose(0, 1)
        (o_ref.float() * do.float()).sum().backward()
        rows = zigzag_rows(cp, rank, s // (2 * cp))
        ql = q[rows].clone().requires_grad_(True)
        kvl = torch.cat([k[rows].reshape(len(rows), b, hk * dh), v[rows].reshape(len(rows), b, hk * dh)], -1).clone().requires_grad_(True)
        o = ZigzagRingAttention.apply(ql, kvl, cg, rank, spec.get("impl", "nccl"), causal, scale, hk)
        (o.float() * do[rows].float()).sum().backward()
        tol = lambda t: t.float().abs().max().item() + 1e-6  # noqa: E731
        errs = [(o.float() - o_ref[rows].float()).abs().max().item() / tol(o_ref),
                (ql.grad.float() - qf.grad[rows].float()).abs().max().item() / tol(qf.grad),
                (kvl.grad[..., : hk * dh].reshape(len(rows), b, hk, dh).float() - kf.grad[rows].float()).abs().max().item() / tol(kf.grad),
                (kvl.grad[..., hk * dh:].reshape(len(rows), b, hk, dh).float() - vf.grad[rows].float()).abs().max().item() / tol(vf.grad)]
        worst = max(worst, max(errs))
    t = torch.tensor([worst], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if use_cuda:
        from hetu_galvatron_b200.ops import _lib
        assert _lib.read_error() is None
    if rank == 0:
        print("WORST %.3e" % t.item(), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
