"""Worker of the in-switch all-reduce test: every rank binds a symmetric workspace to an NVSwitch multicast object
(opt-in: GV_ENABLE_MULTICAST=1), runs the ``multimem.ld_reduce`` / ``multimem.st`` all-reduce kernel on a few sizes,
compares with NCCL and leaves in an orderly way (barrier, then the workspaces are released before the process group).
Nothing in this process is made to fail."""
import json
import os
import sys

os.environ["GV_ENABLE_MULTICAST"] = "1"

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from hetu_galvatron_b200.ops import _lib  # noqa: E402
from hetu_galvatron_b200.parallel import fused, symm  # noqa: E402
from hetu_galvatron_b200.parallel.mesh import Mesh  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    mesh = Mesh(world, rank, 1)
    cg = mesh.group("tp", world)
    res = {"world": world}
    for n in (world * 4096, 1 << 20, 16 << 20):
        torch.manual_seed(100 + rank)
        buf = torch.randn(n, device=dev, dtype=torch.bfloat16)
        ref = buf.float().clone()
        dist.all_reduce(ref, group=cg.group)
        try:
            got = fused.allreduce_symm(buf, cg, tag="mm", multimem=True)
        except _lib.KernelError as exc:
            res["unavailable"] = str(exc)
            break
        err = ((got.float() - ref).abs().max() / ref.abs().max()).item()
        res["err_%d" % n] = err
        # timing (CUDA events, max over ranks): in-switch form against the two-shot form on plain peer loads
        for name, mm in (("multimem", True), ("peer", False)):
            for _ in range(3):
                fused.allreduce_symm(buf, cg, tag="mm" if mm else "pl", multimem=mm)
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(5):
                fused.allreduce_symm(buf, cg, tag="mm" if mm else "pl", multimem=mm)
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / 5], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            res["ms_%s_%d" % (name, n)] = t.item()
    res["kernel_error"] = _lib.read_error()
    torch.cuda.synchronize()
    dist.barrier()
    symm._WORKSPACES.clear()          # unbind / unmap while every rank is still alive
    import gc
    gc.collect()
    torch.cuda.synchronize()
    dist.barrier()
    if rank == 0:
        print("LOSSES " + json.dumps(res), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
