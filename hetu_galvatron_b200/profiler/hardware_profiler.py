"""Hardware profiler: NVLink/NVSwitch bandwidth and latency tables + the compute/communication overlap coefficient.

Writes the files the search engine reads, with the reference's names and keys
(galvatron/core/profiler/hardware_profiler.py:184-315,490-500):

* ``allreduce_bandwidth_{N}nodes_{G}gpus_per_node.json``  ``{"allreduce_size_{k}_consec_{0|1}": bus GB/s}``
* ``p2p_bandwidth_{N}nodes_{G}gpus_per_node.json``        ``{"pp_size_{k}": GB/s}``
* ``sp_time_{N}nodes_{G}gpus_per_node.json``              ``{"allreduce_size_{k}_{m}MB_time": ms, "all2all_size_{k}_{m}MB_time": ms}``
* ``overlap_coefficient.json``                            ``{"overlap_coe": >= 1.0}``

The reference shells out to nccl-tests / mpirun and parses their stdout; here every measurement runs inside the
already-initialised ``torch.distributed`` job (one process per GPU), is timed with CUDA events on the device and
reduced as the max over ranks. ``--backend native`` (the default; the reference's choices are nccl / torch) times this
package's own peer-memory kernels for the tables the search engine reads -- two-shot all-reduce, one-sided send/recv,
pull all-to-all (csrc/nvlink_bench.cu) -- instead of the vendored nccl-tests binaries of the reference;
``--backend nccl`` times the NCCL collectives. Either way a summary of the own kernels (pull all-gather, in-switch
all-reduce when a multicast mapping exists) goes to ``nvlink_native_{N}nodes_{G}gpus_per_node.json``.
"""
from __future__ import annotations

import os
import subprocess
import sys
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..utils.config_utils import write_json_config


def _event_time_ms(fn, iters: int, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def _max_over(group, value: float, device) -> float:
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


class HardwareProfiler:
    def __init__(self, args):
        self.args = args
        self.path = None

    def set_path(self, path: str) -> None:
        self.path = path

    def config_dir(self) -> str:
        d = os.path.join(self.path or os.getcwd(), "hardware_configs")
        os.makedirs(d, exist_ok=True)
        return d

    def _tag(self) -> str:
        return "%dnodes_%dgpus_per_node.json" % (self.args.num_nodes, self.args.num_gpus_per_node)

    # ------------------------------------------------------------------ group enumeration (all ranks, same order)
    @staticmethod
    def group_ranks(world: int, size: int, consecutive: bool) -> List[List[int]]:
        """All groups of ``size`` ranks: consecutive blocks, or strided by world/size (reference :380-420)."""
        if consecutive:
            return [list(range(b * size, (b + 1) * size)) for b in range(world // size)]
        stride = world // size
        return [list(range(o, world, stride)) for o in range(stride)]

    def _make_groups(self, world: int, size: int, consecutive: bool):
        mine = None
        rank = dist.get_rank()
        for ranks in self.group_ranks(world, size, consecutive):
            g = dist.new_group(ranks) if size < world else dist.group.WORLD
            if rank in ranks:
                mine = g
        return mine

    # ------------------------------------------------------------------ own kernels as the measured backend
    def _native(self) -> bool:
        """True when the tables are to be measured with this package's peer-memory kernels and those can run here."""
        if getattr(self.args, "backend", "native") != "native":
            return False
        if getattr(self, "_native_ok", None) is None:
            from ..parallel import symm
            from ..parallel.mesh import Mesh

            self._mesh = Mesh(dist.get_world_size(), dist.get_rank(), 1)
            self._native_ok = symm.available(self._mesh.group("tp", dist.get_world_size())) if dist.get_world_size() > 1 else False
        return self._native_ok

    def _native_group(self, size: int, consecutive: bool):
        """CommGroup of ``size`` ranks holding this rank: consecutive block, or strided by world / size."""
        world = dist.get_world_size()
        return self._mesh.group("tp", size) if consecutive or size == world else self._mesh.group("wdp", world // size)

    # ------------------------------------------------------------------ measurements
    def profile_allreduce_bandwidth(self, size_mb: int = 256, iters: int = 10) -> Dict[str, float]:
        world, dev = dist.get_world_size(), torch.device("cuda", torch.cuda.current_device())
        out = {}
        size = world
        first = True
        while size >= 2:
            for consec in ([1] if first else [0, 1]):
                if self._native():
                    from ..parallel import fused
                    cg = self._native_group(size, bool(consec))
                    buf = torch.empty(size_mb * 2 ** 20 // 2, dtype=torch.bfloat16, device=dev).normal_()
                    ms = _event_time_ms(lambda: fused.allreduce_symm(buf, cg, "hw%d_%d" % (size, consec)), iters)
                else:
                    group = self._make_groups(world, size, bool(consec))
                    buf = torch.empty(size_mb * 2 ** 20 // 4, dtype=torch.float32, device=dev)
                    ms = _event_time_ms(lambda: dist.all_reduce(buf, group=group), iters)
                ms = _max_over(dist.group.WORLD, ms, dev)
                algbw = size_mb / 1024 / (ms / 1e3)
                out["allreduce_size_%d_consec_%d" % (size, consec)] = round(algbw * 2 * (size - 1) / size, 3)
                del buf
            first = False
            size //= 2
        return out

    def profile_p2p_bandwidth(self, size_mb: int = 256, iters: int = 10) -> Dict[str, float]:
        world, rank = dist.get_world_size(), dist.get_rank()
        dev = torch.device("cuda", torch.cuda.current_device())
        out = {}
        pp = 2
        while pp <= min(world, self.args.max_pp_deg):
            stage = world // pp
            buf = torch.empty(size_mb * 2 ** 20 // 2, dtype=torch.bfloat16, device=dev)
            nxt, prv = rank + stage, rank - stage

            def step():
                ops = []
                if nxt < world:
                    ops.append(dist.P2POp(dist.isend, buf, nxt))
                if prv >= 0:
                    ops.append(dist.P2POp(dist.irecv, buf, prv))
                for r in dist.batch_isend_irecv(ops) if ops else []:
                    r.wait()

            if self._native():
                from ..parallel import fused
                cg = self._native_group(world, True)
                # one-sided: every rank pulls the buffer of the rank one stage before it (the first stage wraps around)
                step = lambda: fused.p2p_pull(buf, (rank - stage) % world, cg, "hwpp%d" % pp)   # noqa: E731
            ms = _max_over(dist.group.WORLD, _event_time_ms(step, iters), dev)
            out["pp_size_%d" % pp] = round(size_mb / 1024 / (ms / 1e3), 3)
            pp *= 2
        return out

    def profile_sp_time(self, start_mb: int = 1, end_mb: int = 1024, iters: int = 5) -> Dict[str, float]:
        world, dev = dist.get_world_size(), torch.device("cuda", torch.cuda.current_device())
        out = {}
        size = world
        while size >= 2:
            native = self._native()
            group = None if native else self._make_groups(world, size, True)
            cg = self._native_group(size, True) if native else None
            mb = start_mb
            while mb <= end_mb:
                n = mb * 2 ** 20 // 2
                buf = torch.empty(n, dtype=torch.bfloat16, device=dev).normal_()
                dst = torch.empty(n, dtype=torch.bfloat16, device=dev)
                if native:
                    from ..parallel import fused
                    ar = lambda: fused.allreduce_symm(buf, cg, "hwsp%d" % size)          # noqa: E731
                    a2a = lambda: fused.alltoall_pull(buf, cg, "hwsp%d" % size)          # noqa: E731
                else:
                    ar = lambda: dist.all_reduce(buf, group=group)                       # noqa: E731
                    a2a = lambda: dist.all_to_all_single(dst, buf, group=group)          # noqa: E731
                ms = _max_over(dist.group.WORLD, _event_time_ms(ar, iters), dev)
                out["allreduce_size_%d_%dMB_time" % (size, mb)] = ms
                ms = _max_over(dist.group.WORLD, _event_time_ms(a2a, iters), dev)
                out["all2all_size_%d_%dMB_time" % (size, mb)] = ms
                del buf, dst
                mb *= 2
            size //= 2
        return out

    def profile_overlap(self, iters: int = 20) -> Dict[str, float]:
        """Slow-down of a GEMM stream and an all-reduce stream when they run together (reference
        profile_overlap.py:146-185: overlap_coe = max(comm slow-down, compute slow-down))."""
        from ..ops.gemm import gemm

        dev = torch.device("cuda", torch.cuda.current_device())
        a = torch.randn(8192, 4096, device=dev, dtype=torch.bfloat16)
        w = torch.randn(4096, 4096, device=dev, dtype=torch.bfloat16)
        buf = torch.empty(4096 * 4096, dtype=torch.float32, device=dev)
        comm_stream = torch.cuda.Stream()
        reps = max(self.args.overlap_time_multiply, 1) * 4

        def compute():
            for _ in range(reps):
                gemm(a, w)

        def comm():
            with torch.cuda.stream(comm_stream):
                for _ in range(reps):
                    dist.all_reduce(buf)

        def both():
            comm_stream.wait_stream(torch.cuda.current_stream())
            comm()
            compute()
            torch.cuda.current_stream().wait_stream(comm_stream)

        def comm_only():
            comm_stream.wait_stream(torch.cuda.current_stream())
            comm()
            torch.cuda.current_stream().wait_stream(comm_stream)

        t_comp = _max_over(dist.group.WORLD, _event_time_ms(compute, iters), dev)
        t_comm = _max_over(dist.group.WORLD, _event_time_ms(comm_only, iters), dev)
        t_both = _max_over(dist.group.WORLD, _event_time_ms(both, iters), dev)
        coe = max(t_both / max(t_comp, t_comm), 1.0)
        return {"overlap_coe": round(coe, 4), "compute_ms": t_comp, "comm_ms": t_comm, "together_ms": t_both}

    def profile_native(self, sizes_mb=(16, 64, 256)) -> Dict[str, float]:
        """What this package's own peer-memory kernels reach over NVSwitch (csrc/nvlink_bench.cu, csrc/comm_kernels.cu):
        pull all-gather, one-sided send/recv, all-to-all and two-shot all-reduce (plain peer loads, and the in-switch
        ``multimem`` form when the workspace has a multicast mapping). GB/s are per GPU, inbound, for the gathers and
        copies; bus bandwidth (2 (n-1)/n x size / time) for the all-reduce, like the NCCL table."""
        from ..parallel import fused
        from ..parallel.mesh import Mesh

        world, rank = dist.get_world_size(), dist.get_rank()
        dev = torch.device("cuda", torch.cuda.current_device())
        mesh = Mesh(world, rank, 1)
        cg = mesh.group("tp", world)
        out = {}
        for mb in sizes_mb:
            n = mb * 2 ** 20 // 2
            shard = torch.empty(n, dtype=torch.bfloat16, device=dev)
            dst = torch.empty(world * n, dtype=torch.bfloat16, device=dev)
            ms = _max_over(dist.group.WORLD, _event_time_ms(lambda: fused.allgather_pull(shard, cg, "bench", out=dst), 5), dev)
            out["allgather_pull_%dMB_per_rank_GBps_in" % mb] = round(mb * (world - 1) / 1024 / (ms / 1e3), 2)
            ms = _max_over(dist.group.WORLD, _event_time_ms(lambda: fused.p2p_pull(shard, (rank + 1) % world, cg, "bench"), 5), dev)
            out["p2p_pull_%dMB_GBps" % mb] = round(mb / 1024 / (ms / 1e3), 2)
            ms = _max_over(dist.group.WORLD, _event_time_ms(lambda: fused.alltoall_pull(shard, cg, "bench"), 5), dev)
            out["all2all_pull_%dMB_time" % mb] = ms
            shard.normal_()
            ms = _max_over(dist.group.WORLD, _event_time_ms(lambda: fused.allreduce_symm(shard, cg, "bench"), 5), dev)
            out["allreduce_twoshot_%dMB_busbw" % mb] = round(mb / 1024 / (ms / 1e3) * 2 * (world - 1) / world, 2)
            out["allreduce_twoshot_%dMB_time" % mb] = ms
            try:
                ms = _max_over(dist.group.WORLD, _event_time_ms(lambda: fused.allreduce_symm(shard, cg, "benchmm", multimem=True), 5), dev)
                out["allreduce_multimem_%dMB_busbw" % mb] = round(mb / 1024 / (ms / 1e3) * 2 * (world - 1) / world, 2)
            except Exception as exc:
                out.setdefault("allreduce_multimem", "unavailable: " + str(exc)[:120])
            del shard, dst
        return out

    # ------------------------------------------------------------------ drivers
    def profile_all(self, native: bool = True, only: Optional[List[str]] = None) -> Dict[str, dict]:
        """Run the measurements (all, or those named in ``only``: allreduce, p2p, sp, overlap, native) in this already
        distributed job and write their JSON files from rank 0."""
        a = self.args
        want = set(only or ["allreduce", "p2p", "sp", "overlap"] + (["native"] if native else []))
        res: Dict[str, dict] = {}
        if "allreduce" in want:
            res["allreduce"] = self.profile_allreduce_bandwidth()
        if "p2p" in want:
            res["p2p"] = self.profile_p2p_bandwidth()
        if "sp" in want:
            res["sp"] = self.profile_sp_time(max(a.start_mb, 1) if a.start_mb < 16 else 1, 1024)
        if "overlap" in want:
            res["overlap"] = self.profile_overlap()
        if "native" in want:
            try:
                res["native"] = self.profile_native()
            except Exception as exc:  # symmetric memory unavailable: keep the NCCL tables
                res["native"] = {"unavailable": str(exc)[:200]}
        if dist.get_rank() == 0:
            d = self.config_dir()
            files = {"allreduce": "allreduce_bandwidth_" + self._tag(), "p2p": "p2p_bandwidth_" + self._tag(),
                     "sp": "sp_time_" + self._tag(), "overlap": "overlap_coefficient.json", "native": "nvlink_native_" + self._tag()}
            for key, table in res.items():
                write_json_config({"overlap_coe": table["overlap_coe"]} if key == "overlap" else table, os.path.join(d, files[key]))
        return res

    # names kept from the reference's driver API
    def profile_bandwidth(self, backend: str = "native"):
        return {"allreduce": self.profile_allreduce_bandwidth(), "p2p": self.profile_p2p_bandwidth()}

    def profile_sp_bandwidth(self, backend: str = "native"):
        return self.profile_sp_time()

    def launch(self, script: str, extra: Optional[List[str]] = None) -> int:
        """Start ``script`` under torchrun on this node's GPUs (used when the caller is a plain process)."""
        a = self.args
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=%d" % a.num_nodes,
               "--nproc-per-node", str(a.num_gpus_per_node), "--master-addr", "127.0.0.1", "--master-port", "29561", script]
        return subprocess.call(cmd + (extra or []))


def main(argv=None):
    """``python -m torch.distributed.run --nproc-per-node G --master-addr 127.0.0.1 -m
    hetu_galvatron_b200.profiler.hardware_profiler [--num_gpus_per_node G ...]``: measures inside this job and writes
    the tables under ``<--output_dir or hetu_galvatron_b200/profile_hardware>/hardware_configs`` (reference entry: galvatron/profile_hardware/
    profile_hardware.py + scripts/profile_hardware.sh, which generate and run nccl-tests scripts)."""
    import argparse

    from .arguments import galvatron_profile_hardware_args

    ap = galvatron_profile_hardware_args(argparse.ArgumentParser())
    ap.add_argument("--output_dir", type=str, default=None)
    ap.add_argument("--no_native", action="store_true", help="skip this package's own peer-memory kernels")
    ap.add_argument("--only", type=str, nargs="+", default=None, choices=["allreduce", "p2p", "sp", "overlap", "native"],
                    help="measure only these tables")
    args = ap.parse_args(argv)
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl")
    args.num_gpus_per_node = min(args.num_gpus_per_node, dist.get_world_size())
    args.num_nodes = max(1, dist.get_world_size() // args.num_gpus_per_node)
    prof = HardwareProfiler(args)
    pkg = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    prof.set_path(args.output_dir or os.path.join(pkg, "profile_hardware"))     # where the search engine looks by default
    res = prof.profile_all(native=not args.no_native, only=args.only)
    if rank == 0:
        import json
        print("HARDWARE_PROFILE " + json.dumps(res), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
