"""Per-iteration time and memory instrumentation of a training loop.

Same hook points and outputs as the reference's ``RuntimeProfiler``
(galvatron/core/profiler/runtime_profiler.py:99-186 memory, :189-301 time, :303-339 iteration line), with two
differences: the iteration time is taken from CUDA events on the training stream and reduced as the MAX over
ranks (the reference reports the last rank's own time), and every iteration is also appended to a JSONL file
(step time, tokens/s, loss, grad norm, memory) when ``log_path`` is set. On CPU ranks wall-clock time is used.
"""
from __future__ import annotations

import json
import os
import time
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..utils.memory_utils import memory_stats_mb
from .utils import save_profiled_memory, save_profiled_time


class RuntimeProfiler:
    def __init__(self, args, path: Optional[str] = None, model_name: Optional[str] = None, log_path: Optional[str] = None):
        self.args = args
        self.path = path
        self.model_name = model_name
        self.log_path = log_path
        self.layernum_list = self.seqlen_list = self.hiddensize_list = None
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world_size = dist.get_world_size() if dist.is_initialized() else 1
        self.mem_dict: Dict[str, float] = {}
        self.profile_ranks: List[int] = [self.rank]
        self.max_profile_iter = 5
        self.start_iter, self.end_iter, self.exit = 10, 20, False
        self.time_list: List[float] = []
        self._t0 = None
        self._ev = None
        self.total_start_time = None
        self.tokens_per_iter = None

    # ------------------------------------------------------------------ configuration
    def set_profiler_dist(self, path=None, model_layer_configs=None, model_name=None, profile_ranks=None, start_iter=10,
                          end_iter=20, rank=None):
        """Distributed set-up: profile memory on the first and last rank, time everywhere (reference :24-48)."""
        rank = self.rank if rank is None else rank
        if profile_ranks is None:
            profile_ranks = [0, self.world_size - 1]
        self.set_model_layer_configs(model_layer_configs)
        self.path = path or self.path
        self.model_name = model_name or self.model_name
        self.set_memory_profiler(rank, profile_ranks)
        exit_ = getattr(self.args, "exit_after_profiling", True)
        self.set_time_profiler(start_iter=start_iter, end_iter=end_iter, exit=bool(exit_))

    def set_profiler_single(self, start_iter=10, end_iter=20):
        self.set_memory_profiler(0)
        self.set_time_profiler(start_iter=start_iter, end_iter=end_iter, exit=bool(getattr(self.args, "exit_after_profiling", True)))

    def set_model_layer_configs(self, model_layer_configs) -> None:
        if model_layer_configs is None:
            return
        self.hiddensize_list = [c["hidden_size"] for c in model_layer_configs]
        self.layernum_list = [c["layer_num"] for c in model_layer_configs]
        self.seqlen_list = [c["seq_len"] for c in model_layer_configs]

    def _config_file(self, kind: str) -> str:
        assert self.model_name is not None, "Should specify the model name!"
        name = "%s_profiling_%s_%s.json" % (kind, getattr(self.args, "mixed_precision", "bf16"), self.model_name)
        return os.path.join(self.path, "configs", name)

    def memory_profiling_path(self) -> str:
        return self._config_file("memory")

    def time_profiling_path(self) -> str:
        return self._config_file("computation")

    # ------------------------------------------------------------------ memory
    def set_memory_profiler(self, rank: int, profile_ranks: List[int] = [], max_profile_iter: int = 5) -> None:
        self.rank = rank
        self.profile_ranks = list(profile_ranks) if len(profile_ranks) > 0 else [rank]
        self.mem_dict = {}
        self.max_profile_iter = max_profile_iter

    def _mem(self):
        kind = getattr(self.args, "profile_type", "allocated")
        s = memory_stats_mb(getattr(self.args, "local_rank", None) if torch.cuda.is_available() else None)
        return (s["max_allocated"], s["allocated"]) if kind == "allocated" else (s["max_reserved"], s["reserved"])

    def profile_memory(self, iter: int, stage: str = "") -> None:
        if not getattr(self.args, "profile", 0) or self.rank not in self.profile_ranks or iter is None or iter > self.max_profile_iter:
            return
        if stage == "Before Forward" and torch.cuda.is_available():
            torch.cuda.reset_peak_memory_stats()
        peak, cur = self._mem()
        tag = {"Before Forward": "before_forward", "After Forward": "after_forward", "After Backward": "after_backward"}.get(stage)
        print("%s\n\tMax memory: %.2f MB\tCurrent memory : %.2f MB" % (stage, peak, cur))
        if tag is None:
            return
        self.mem_dict["iter_%d_%s" % (iter, tag)] = cur
        if tag == "after_backward":
            self.mem_dict["iter_%d_after_backward_max" % iter] = peak

    def post_profile_memory(self, iter: int) -> None:
        args = self.args
        if not getattr(args, "profile", 0) or iter != self.max_profile_iter:
            return
        if self.rank in self.profile_ranks:
            m, k = self.mem_dict, self.max_profile_iter - 1
            m["model_states"] = m.get("iter_%d_after_backward" % k, 0.0)
            if getattr(args, "pipeline_type", "gpipe") == "gpipe" and ("iter_%d_after_forward" % k) in m:
                m["model_states_and_activation"] = m["iter_%d_after_forward" % k]
                m["activation"] = m["iter_%d_after_forward" % k] - m["iter_%d_before_forward" % k]
            m["model_states_and_peak_activation"] = m.get("iter_%d_after_backward_max" % k, 0.0)
            m["peak_activation"] = m["model_states_and_peak_activation"] - m["model_states"]
            m.setdefault("activation", m["peak_activation"])
            print("[Profiled memory for rank %d]:" % self.rank)
            for key, val in m.items():
                print("\t%s: %.2f MB" % (key, val))
        if getattr(args, "save_profiled_memory", 0):
            # one writer: the profiled ranks hand their figures to rank 0 (two ranks rewriting the same JSON file
            # at the same moment lose entries)
            mine = None
            if self.rank in self.profile_ranks:
                m = self.mem_dict
                mine = (self.rank, m["model_states"], m["activation"], m["peak_activation"])
            entries = [mine]
            if dist.is_initialized() and self.world_size > 1:
                entries = [None] * self.world_size
                dist.all_gather_object(entries, mine)
            if self.rank == 0:
                assert self.layernum_list is not None
                for e in entries:
                    if e is not None:
                        save_profiled_memory(self.memory_profiling_path(), args.pp_deg, args.global_tp_deg, self.world_size,
                                             self.layernum_list, args.global_train_batch_size, e[0], e[1], e[2], e[3],
                                             getattr(args, "global_checkpoint", 0), getattr(args, "sequence_parallel", False),
                                             getattr(args, "vocab_tp", 1), self.seqlen_list)
            if dist.is_initialized() and self.world_size > 1:
                dist.barrier()
        if getattr(args, "save_profiled_memory", 0):
            raise SystemExit(0)

    # ------------------------------------------------------------------ time
    def set_time_profiler(self, start_iter: int, end_iter: int, exit: bool = False) -> None:
        assert end_iter > start_iter, "End iteration must be greater than start iteration"
        self.start_iter, self.end_iter, self.exit = start_iter, end_iter, exit
        self.time_list = []

    def _sync(self):
        if torch.cuda.is_available():
            torch.cuda.synchronize()

    def profile_time_start(self, iter: int) -> None:
        if not getattr(self.args, "profile", 0):
            return
        if self.total_start_time is None:
            self.total_start_time = time.time()
        if torch.cuda.is_available():
            self._sync()
            self._ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            self._ev[0].record()
        self._t0 = time.perf_counter()

    def profile_time_end(self, iter: int, loss=None, learning_rate=None, grad_norm=None) -> None:
        if not getattr(self.args, "profile", 0) or self._t0 is None:
            return
        if torch.cuda.is_available() and self._ev is not None:
            self._ev[1].record()
            self._sync()
            seconds = self._ev[0].elapsed_time(self._ev[1]) / 1e3
        else:
            seconds = time.perf_counter() - self._t0
        seconds = self._max_over_ranks(seconds)
        if self.start_iter <= iter < self.end_iter:
            self.time_list.append(seconds)
        if self.rank == self.world_size - 1:
            self._log_iteration_stats(iter, seconds, loss, learning_rate, grad_norm)
        self._jsonl(iter, seconds, loss, learning_rate, grad_norm)
        if iter == self.end_iter - 1 and self.time_list:
            self._process_time_results()

    def profile_time_python(self, iter: int) -> None:
        """Coarse timing by wall clock, without device synchronisation: mark ``start_iter`` and at ``end_iter`` print (and, for
        forward profiling, store) the mean seconds per iteration in between (reference: runtime_profiler.py:252-277, which
        stores this figure in seconds, unlike the event-timed path)."""
        if not getattr(self.args, "profile", 0):
            return
        if iter == self.start_iter:
            self.total_start_time = time.time()
        elif iter == self.end_iter:
            self.total_end_time = time.time()
            avg = (self.total_end_time - self.total_start_time) / (self.end_iter - self.start_iter)
            print("Average iteration time is: %.4f s" % avg)
            if getattr(self.args, "profile_forward", 0):
                assert self.layernum_list is not None
                save_profiled_time(self.time_profiling_path(), avg, self.args.global_train_batch_size, self.layernum_list, self.seqlen_list)
            if self.exit:
                exit(0)

    def profile_optimizer_start(self) -> None:
        """Bracket the optimizer step (+ zero_grad) of the iterations whose whole-iteration time is being stored, so that
        the model profiler can separate the per-iteration optimizer cost from the per-micro-batch backward cost."""
        if not (getattr(self.args, "profile", 0) and getattr(self.args, "save_profiled_iteration", 0)) or not torch.cuda.is_available():
            return
        self._opt_ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        self._opt_ev[0].record()

    def profile_optimizer_end(self, iter: int) -> None:
        ev = getattr(self, "_opt_ev", None)
        if ev is None:
            return
        ev[1].record()
        self._opt_ev = None
        if self.start_iter <= iter < self.end_iter:
            self._opt_events = getattr(self, "_opt_events", []) + [ev]

    def _max_over_ranks(self, seconds: float) -> float:
        if self.world_size == 1 or not dist.is_initialized():
            return seconds
        dev = torch.device("cuda") if (torch.cuda.is_available() and dist.get_backend() == "nccl") else torch.device("cpu")
        t = torch.tensor([seconds], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def _process_time_results(self) -> None:
        avg = sum(self.time_list) / len(self.time_list)
        print("Average iteration time is: %.4f s" % avg)
        self.last_average_time = avg
        if getattr(self.args, "profile_forward", 0):
            assert self.layernum_list is not None
            save_profiled_time(self.time_profiling_path(), avg * 1e3, self.args.global_train_batch_size, self.layernum_list,
                               self.seqlen_list)
        elif getattr(self.args, "save_profiled_iteration", 0) and self.rank == 0:
            assert self.layernum_list is not None
            save_profiled_time(self.time_profiling_path(), avg * 1e3, self.args.global_train_batch_size, self.layernum_list,
                               self.seqlen_list, suffix="_iter")
            evs = getattr(self, "_opt_events", [])
            if evs:
                self._sync()
                opt_ms = sum(a.elapsed_time(b) for a, b in evs) / len(evs)
                save_profiled_time(self.time_profiling_path(), opt_ms, self.args.global_train_batch_size, self.layernum_list,
                                   self.seqlen_list, suffix="_opt")
                self._opt_events = []
        if self.exit:
            raise SystemExit(0)
        span = self.end_iter - self.start_iter
        self.time_list = []
        self.start_iter, self.end_iter = self.end_iter, self.end_iter + span

    def _log_iteration_stats(self, iter, iter_time, loss, learning_rate, grad_norm) -> None:
        if loss is None:
            print(iter_time)
            return
        print("| Iteration: {:6d} | Consumed samples: {:12d} | Elapsed time per iteration (ms): {:.1f} | "
              "Learning rate: {:.6e} | Loss: {:.6e} | grad norm: {:.2f} |".format(
                  iter + 1, (iter + 1) * self.args.global_train_batch_size, iter_time * 1e3,
                  getattr(self.args, "lr", 0.0) if learning_rate is None else learning_rate, float(loss),
                  0.0 if grad_norm is None else float(grad_norm)), flush=True)

    def _jsonl(self, iter, seconds, loss, lr, grad_norm) -> None:
        if not self.log_path:
            return
        rec = {"iter": iter, "rank": self.rank, "step_time_s_max_over_ranks": seconds,
               "loss": None if loss is None else float(loss), "lr": lr,
               "grad_norm": None if grad_norm is None else float(grad_norm)}
        if self.tokens_per_iter:
            rec["tokens_per_s"] = self.tokens_per_iter / seconds
        rec.update({"mem_" + k: v for k, v in memory_stats_mb().items()})
        os.makedirs(os.path.dirname(self.log_path) or ".", exist_ok=True)
        with open("%s.rank%d.jsonl" % (self.log_path, self.rank), "a") as fp:
            fp.write(json.dumps(rec) + "\n")
