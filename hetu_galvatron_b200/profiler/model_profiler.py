"""Model profiler: per-layer forward time and per-layer / other memory, in the reference's profile-file grammar.

The reference (galvatron/core/profiler/model_profiler.py) drives ``os.system`` launches of a training script per
measurement point and post-processes the raw keys the runtime profiler wrote:

* computation (:223-252, :328-372): forward time of models with ``layernum_min`` and ``layernum_max`` layers per
  layer type -> ``layertype_{i}_bsz{B}_seq{S}`` = ms per layer per sample, ``layertype_other_bsz{B}_seq{..}``.
* memory (:175-221, :374-700): model-state and activation MB of (pp, tp, checkpoint, vocab-tp) configurations ->
  ``layertype_{i}[_sp]`` = {seq: {parameter_size, tp_activation_per_bsz_dict}} and ``other_memory_pp_{off,on_first,
  on_last}[_sp]`` = {seq: {model_states: {tp: MB}, activation: {tp: MB}}}.

This implementation separates the three concerns: ``*_points()`` enumerate the measurement points as plain dicts
(testable without a GPU), ``launch_profiling_scripts()`` runs them (in this process for single-GPU computation
points, as ``torch.distributed.run`` jobs otherwise), and ``process_profiled_data()`` derives the search engine's keys.
"""
from __future__ import annotations

import copy
import os
import shlex
import subprocess
import sys
from itertools import product
from typing import Dict, List, Optional, Sequence, Tuple

from ..utils.config_utils import array2str, num2str, read_json_config, str2array, write_json_config

INF_MB = 1e6

# flags of the profiler itself: never forwarded to the training script
_OWN_FLAGS = {
    "profile_type", "set_model_config_manually", "set_layernum_manually", "set_seqlen_manually",
    "profile_batch_size", "profile_min_batch_size", "profile_max_batch_size", "profile_batch_size_step",
    "profile_seq_length_list", "profile_min_seq_length", "profile_max_seq_length", "profile_seq_length_step",
    "layernum_min", "layernum_max", "max_tp_deg", "profile_dp_type", "mixed_precision", "use_flash_attn",
    "sequence_parallel", "extra_args_str", "seq_length", "encoder_seq_length", "decoder_seq_length", "in_process",
    "shape_order", "make_vocab_size_divisible_by", "galvatron_mode", "local_rank",
}


def raw_key(layernum, bsz=None, seq=None, rank=None, kind=None) -> str:
    """``layernum[1,2]_bsz8_seq512_rank0_ms`` (reference key_format :702-739)."""
    s = "layernum[%s]" % array2str(layernum) if isinstance(layernum, (list, tuple)) else "layernum%s" % layernum
    if bsz is not None:
        s += "_bsz%d" % bsz
    if seq is not None:
        s += "_" + seq if isinstance(seq, str) else "_seq%d" % seq
    if rank is not None and kind is not None:
        s += "_rank%d_%s" % (rank, kind)
    return s


def stage_cost(pp_deg: int, layernum: int, per_type_cost: Sequence[float], stage: int) -> float:
    """Sum of per-layer costs of the layers an even pipeline split puts on ``stage`` (layer types in order,
    ``layernum`` layers each)."""
    costs = [c for c in per_type_cost for _ in range(layernum)]
    per = len(costs) // pp_deg
    assert per * pp_deg == len(costs), "profiling configurations divide evenly over the stages"
    return float(sum(costs[stage * per:(stage + 1) * per]))


class ModelProfiler:
    def __init__(self, args):
        self.args = args
        self.path: Optional[str] = None
        self.model_name: Optional[str] = None
        self.layernum_arg_names: List[str] = []
        self.layernum_listed = False
        self.seqlen_arg_names: Optional[List[str]] = ["seq_length"]
        self.num_layertype = 1
        self.sequence_length_list: List[List[int]] = []
        self.family = "llama"  # model family of the in-process runs
        self._launches = 0
        self.runner = None     # injectable: callable(point dict) -> None, replaces the subprocess launch (tests)

    # ------------------------------------------------------------------ configuration
    def set_path(self, path: str) -> None:
        self.path = path

    def set_model_name(self, name: str) -> None:
        self.model_name = name

    def _profile_file(self, kind: str) -> str:
        assert self.model_name is not None, "Should specify the model name!"
        name = "%s_profiling_%s_%s.json" % (kind, self.args.mixed_precision, self.model_name)
        d = os.path.join(self.path, "configs")
        os.makedirs(d, exist_ok=True)
        return os.path.join(d, name)

    def memory_profiling_path(self) -> str:
        return self._profile_file("memory")

    def time_profiling_path(self) -> str:
        return self._profile_file("computation")

    def set_profiler_launcher(self, path: str, layernum_arg_names: Optional[List[str]] = None, model_name: Optional[str] = None,
                              seqlen_arg_names: Optional[List[str]] = None, layernum_listed: bool = False) -> None:
        self.set_path(path)
        self.set_model_name(model_name)
        self.layernum_arg_names = list(layernum_arg_names or [])
        self.layernum_listed = layernum_listed
        if layernum_listed:      # one list-valued flag (Swin ``depths``): one layer type per entry
            assert len(self.layernum_arg_names) == 1
            self.num_layertype = len(getattr(self.args, self.layernum_arg_names[0]))
        else:
            self.num_layertype = len(self.layernum_arg_names)
        self.seqlen_arg_names = ["seq_length"] if seqlen_arg_names is None else seqlen_arg_names
        self._resolve_sequence_lengths()

    def _resolve_sequence_lengths(self) -> None:
        a, T = self.args, self.num_layertype
        if a.profile_seq_length_list is not None:
            base = str2array(a.profile_seq_length_list) if isinstance(a.profile_seq_length_list, str) else list(a.profile_seq_length_list)
            assert len(base) == T, "one profile sequence length per layer type"
        elif self.layernum_listed:
            base = [(a.image_size // a.patch_size // (2 ** i)) ** 2 for i in range(T)]
        else:
            base = [getattr(a, "seq_length", None) or 2048] * T
        self.profile_seq_length_list = base
        if a.profile_mode in ("static", "batch"):
            self.sequence_length_list = [[s] for s in base]
            return
        assert T == 1, "Sequence profiling only support single layertype!"
        lo, hi = a.profile_min_seq_length, a.profile_max_seq_length
        assert lo is not None and hi is not None
        if a.profile_type == "computation":
            self.sequence_length_list = [list(range(lo, hi + 1, a.profile_seq_length_step))]
        else:
            assert lo & (lo - 1) == 0 and hi & (hi - 1) == 0, "memory profiling wants power-of-two sequence lengths"
            self.sequence_length_list = [[1 << j for j in range(lo.bit_length() - 1, hi.bit_length())]]

    def set_seqlen_list(self) -> None:
        """The reference's name for this step (model_profiler.py:77-130)."""
        self._resolve_sequence_lengths()

    # ------------------------------------------------------------------ enumeration of measurement points
    def layernum_lists(self) -> List[List[int]]:
        """[min]*T followed by, for every layer type, the list with that type at ``layernum_max``."""
        a = self.args
        base = [a.layernum_min] * self.num_layertype
        out = [base]
        for t in range(self.num_layertype):
            l = list(base)
            l[t] = a.layernum_max
            out.append(l)
        return out

    def get_bsz_list(self) -> List[int]:
        a = self.args
        if a.profile_mode == "batch":
            assert a.profile_min_batch_size is not None and a.profile_max_batch_size is not None
            return list(range(a.profile_min_batch_size, a.profile_max_batch_size + 1, a.profile_batch_size_step))
        assert a.profile_batch_size is not None
        return [a.profile_batch_size]

    def seq_tuples(self) -> List[Tuple[int, ...]]:
        return list(product(*self.sequence_length_list))

    def world_size(self) -> int:
        if self.args.profile_type != "memory":
            return 1
        return int(os.getenv("NUM_NODES", "1")) * int(os.getenv("NUM_GPUS_PER_NODE", "8"))

    def _layer_flags(self, layernums: Sequence[int], seq: Sequence[int]) -> Dict[str, object]:
        f: Dict[str, object] = {}
        if self.layernum_listed:
            f[self.layernum_arg_names[0]] = list(layernums)
        else:
            f.update(dict(zip(self.layernum_arg_names, layernums)))
        if self.seqlen_arg_names:
            f.update(dict(zip(self.seqlen_arg_names, seq)))
        return f

    def computation_points(self) -> List[Dict[str, object]]:
        pts = []
        for layernums in self.layernum_lists():
            for bsz in self.get_bsz_list():
                for seq in self.seq_tuples():
                    p = self._layer_flags(layernums, seq)
                    p.update(pp_deg=1, global_tp_deg=1, global_checkpoint=0, global_train_batch_size=bsz)
                    pts.append(p)
        if self.args.profile_mode == "static" and getattr(self.args, "profile_iteration", 1):
            # whole iterations (forward + backward + optimizer step) of the smallest and the first varied model:
            # their per-layer slope against the forward slope is the measured backward / forward ratio
            lists = self.layernum_lists()
            for layernums in (lists[0], lists[1]):
                p = self._layer_flags(layernums, self.seq_tuples()[0])
                p.update(pp_deg=1, global_tp_deg=1, global_checkpoint=0, global_train_batch_size=self.get_bsz_list()[0],
                         profile_forward=0, save_profiled_iteration=1)
                pts.append(p)
        return pts

    def memory_points(self) -> List[Dict[str, object]]:
        a, world = self.args, self.world_size()
        assert a.profile_mode in ("static", "sequence"), "Memory profiling only supports sequence or static profile mode."
        max_tp = min(world, a.max_tp_deg) if a.profile_mode == "static" else 1
        tps = [t for t in (1, 2, 4, 8, 16) if t <= max_tp]
        pts = []

        def add(layernums, seq, pp, tp, ckpt, vtp):
            p = self._layer_flags(layernums, seq)
            p.update(pp_deg=pp, global_tp_deg=tp, global_checkpoint=ckpt, vocab_tp=tp if vtp else 1,
                     global_train_batch_size=a.profile_batch_size)
            pts.append(p)

        for seq in self.seq_tuples():
            # no pipeline: every tp degree (with and without a tp-sharded vocabulary); checkpointing only at tp 1
            for ckpt in (0, 1):
                for tp in (tps if not ckpt else tps[:1]):
                    if tp > world:
                        continue
                    for vtp in ((0,) if tp == 1 else (0, 1)):
                        for layernums in self.layernum_lists():
                            add(layernums, seq, 1, tp, ckpt, vtp)
            # pipeline on: one layer of every type per stage
            for pp in (2, 4):
                for tp in tps:
                    if pp * tp > world:
                        continue
                    for vtp in ((0,) if tp == 1 else (0, 1)):
                        add([pp] * self.num_layertype, seq, pp, tp, 0, vtp)
        return pts

    def general_flags(self) -> Dict[str, object]:
        """Flags common to every point (reference profiling_general_args :960-993)."""
        a = self.args
        mem = a.profile_type == "memory"
        f: Dict[str, object] = dict(
            set_model_config_manually=0, set_layernum_manually=1, set_seqlen_manually=1, epochs=10, lr=1e-4,
            adam_weight_decay=0.01, dropout_prob=getattr(a, "profile_dropout_prob", 0.0), check_loss=0, profile=1, save_profiled_memory=int(mem),
            profile_forward=int(not mem), initialize_on_meta=1, global_tp_consec=1,
            sdp=int(mem and a.profile_dp_type == "zero3"), chunks=1, pipeline_type="gpipe",
            default_dp_type=a.profile_dp_type if mem else "ddp", mixed_precision=a.mixed_precision, shape_order=a.shape_order)
        if a.use_flash_attn:
            f["use-flash-attn"] = ""
        if a.sequence_parallel:
            f["sequence-parallel"] = ""
        return f

    def model_flags(self) -> Dict[str, object]:
        skip = _OWN_FLAGS | set(self.layernum_arg_names)
        return {k: v for k, v in vars(self.args).items() if k not in skip and v is not None and v is not False and v != ""}

    # ------------------------------------------------------------------ running the points
    @staticmethod
    def flags_to_argv(flags: Dict[str, object]) -> List[str]:
        argv: List[str] = []
        for k, v in flags.items():
            argv.append("--" + k)
            if isinstance(v, (list, tuple)):
                argv.extend(str(x) for x in v)
            elif v != "" and v is not True:
                argv.append(str(v))
        return argv

    def point_argv(self, point: Dict[str, object]) -> List[str]:
        flags = dict(self.model_flags())
        flags.update(self.general_flags())
        flags.update(point)
        argv = self.flags_to_argv(flags)
        for extra in (getattr(self.args, "extra_args_str", "") or "").split("/"):
            if extra:
                argv.extend(("--" + extra).split())
        return argv

    def launch_command(self, point: Dict[str, object]) -> List[str]:
        trainer = os.path.join(self.path, os.getenv("PROFILE_TRAINER", "train_dist_random.py"))
        world = self.world_size()
        if world == 1:
            head = [sys.executable, trainer]
        else:
            launcher = os.getenv("PROFILE_LAUNCHER")
            if launcher:
                head = shlex.split(launcher) + [trainer]
            else:
                head = [sys.executable, "-m", "torch.distributed.run", "--nnodes", os.getenv("NUM_NODES", "1"),
                        "--nproc-per-node", os.getenv("NUM_GPUS_PER_NODE", "8"), "--node-rank", os.getenv("NODE_RANK", "0"),
                        "--master-addr", os.getenv("MASTER_ADDR", "127.0.0.1") or "127.0.0.1",
                        "--master-port", str(int(os.getenv("MASTER_PORT", "29500") or "29500") + self._launches % 64), trainer]
        return head + self.point_argv(point)

    def _run_point(self, point: Dict[str, object]) -> None:
        if self.runner is not None:
            self.runner(point)
            return
        # In-process: single-GPU points always can; multi-GPU points can when this profiler itself runs as one rank of
        # a job of the right size (``torchrun --nproc-per-node G profiler.py --profile_type memory``): every rank then
        # walks the same points, which saves a process start and a rendezvous per point.
        joined = int(os.environ.get("WORLD_SIZE", "1")) == self.world_size() and "RANK" in os.environ
        if getattr(self.args, "in_process", 0) and (self.world_size() == 1 or joined):
            import gc

            import torch

            from ..models import runner as model_runner
            try:
                model_runner.train(self.family, random_data=True, argv=self.point_argv(point))
            except SystemExit:
                pass
            # the next point's figures are absolute allocator readings: nothing of this one may survive
            gc.collect()
            if torch.cuda.is_available():
                torch.cuda.synchronize()
                torch.cuda.empty_cache()
                left = torch.cuda.memory_allocated() / 2 ** 20
                if left > 64:
                    print("warning: %.0f MB still allocated after a profiling point" % left, flush=True)
            return
        cmd = self.launch_command(point)
        self._launches += 1          # consecutive jobs use different rendezvous ports (the previous one may linger)
        print(" ".join(shlex.quote(c) for c in cmd), flush=True)
        subprocess.call(cmd, env=dict(os.environ, CUDA_DEVICE_MAX_CONNECTIONS="1"))

    def launch_profiling_scripts(self) -> None:
        points = self.memory_points() if self.args.profile_type == "memory" else self.computation_points()
        if points and self.args.profile_type == "computation" and getattr(self.args, "in_process", 0) \
                and self.world_size() == 1 and self.runner is None:
            # the first point of a process also pays library start-up, allocator growth and the clock ramp of an idle
            # GPU; the layer time is a DIFFERENCE between points, so the first one is measured a second time afterwards
            self._run_point(points[0])
        for p in points:
            self._run_point(p)

    # ------------------------------------------------------------------ post-processing
    def process_profiled_data(self) -> None:
        if self.args.profile_type == "computation":
            self._process_computation_data()
        else:
            self._process_memory_data()

    def _process_computation_data(self) -> None:
        a, path = self.args, self.time_profiling_path()
        cfg = read_json_config(path)
        lists = self.layernum_lists()
        span = a.layernum_max - a.layernum_min
        for bsz in self.get_bsz_list():
            for seq in self.seq_tuples():
                tag = num2str(list(seq), "seq")
                base = cfg[raw_key(lists[0], bsz, tag)]
                rest = base
                for t, layernums in enumerate(lists[1:]):
                    per_layer_per_sample = (cfg[raw_key(layernums, bsz, tag)] - base) / bsz / span
                    cfg["layertype_%d_bsz%d_seq%d" % (t, bsz, seq[t])] = per_layer_per_sample
                    rest -= lists[0][t] * per_layer_per_sample * bsz
                cfg["layertype_other_bsz%d_%s" % (bsz, tag)] = max(rest / bsz, 0)
                k0, k1 = raw_key(lists[0], bsz, tag) + "_iter", raw_key(lists[1], bsz, tag) + "_iter"
                if k0 in cfg and k1 in cfg:
                    fwd_slope = cfg[raw_key(lists[1], bsz, tag)] - base
                    # the optimizer step (+ zero_grad) runs once per iteration, not once per micro-batch: when it was
                    # timed (keys "_opt"), its per-layer slope is stored on its own and taken out of the ratio
                    o0, o1 = raw_key(lists[0], bsz, tag) + "_opt", raw_key(lists[1], bsz, tag) + "_opt"
                    opt_slope = (cfg[o1] - cfg[o0]) if (o0 in cfg and o1 in cfg) else 0.0
                    if o0 in cfg and o1 in cfg:
                        for t, layernums in enumerate(lists[1:]):
                            ok = raw_key(layernums, bsz, tag) + "_opt"
                            if ok in cfg:
                                cfg["optimizer_ms_layertype_%d" % t] = max((cfg[ok] - cfg[o0]) / span, 0.0)   # per layer and step
                    if fwd_slope > 0:
                        # backward / forward of one layer (with the optimizer folded in when it was not timed apart):
                        # what the cost model multiplies fct by
                        cfg["bct_fct_coe"] = ((cfg[k1] - cfg[k0]) - opt_slope - fwd_slope) / fwd_slope
        write_json_config(cfg, path)
        print("Already written processed computation time into env config file %s!\n" % path)

    def _strategy(self, pp: int, tp: int, world: int, ckpt: bool = False, vtp: bool = False) -> str:
        s = "%d_%d_%d" % (pp, tp, world // pp // tp)
        if ckpt:
            s += "_c"
        if vtp and tp != 1:
            s += "_vtp"
        if self.args.sequence_parallel:
            s += "_sp"
        return s

    def _process_memory_data(self) -> None:
        path = self.memory_profiling_path()
        cfg = read_json_config(path)
        for seq in self.seq_tuples():
            self._process_memory_for_seq(cfg, seq)
        write_json_config(cfg, path)
        print("Already written processed memory into env config file %s!\n" % path)

    def _process_memory_for_seq(self, cfg: dict, seq: Tuple[int, ...]) -> None:
        a, world, T = self.args, self.world_size(), self.num_layertype
        bsz, span, tag = a.profile_batch_size, a.layernum_max - a.layernum_min, num2str(list(seq), "seq")
        lists = self.layernum_lists()
        base, varied = lists[0], lists[1:]
        zero3 = a.profile_dp_type == "zero3"
        tps = [t for t in (1, 2, 4, 8, 16) if t <= world]

        def slope(entry, t, kind):   # MB per extra layer of type t on rank 0
            return (entry[raw_key(varied[t], bsz, tag, 0, kind)] - entry[raw_key(base, bsz, tag, 0, kind)]) / span

        # measured model states -> the 16-bytes-per-parameter unit of the cost model ("4 x parameter_size"). With the
        # 'fsdp' layout a ZeRO-3 rank is taken to hold exactly 1/dp of them (the reference's assumption); with the
        # 'engine' layout the share is what this package's ZeRO engine keeps once an iteration has settled: the
        # full-size gradient buffer stays, the rest is sharded.
        engine_layout = getattr(a, "memory_layout", "fsdp") == "engine"
        mixed = a.mixed_precision != "fp32"

        def share(dp):
            if engine_layout:
                from ..search.cost_model import engine_state_ratio
                return engine_state_ratio("zero3" if zero3 else "ddp", dp, mixed, 4, settled=True)
            return 1.0 / dp if zero3 else 1.0

        # per-layer parameter size (fp32-equivalent MB of ONE copy: model states hold 4 of them) and activation
        # per sample, for every profiled tp degree
        param_by_tp = [dict() for _ in range(T)]
        act_by_tp = [dict() for _ in range(T)]
        param_size = [-1.0] * T
        for tp in tps:
            entry = cfg.get(self._strategy(1, tp, world))
            if entry is None:
                continue
            dp = world // tp
            for t in range(T):
                par = slope(entry, t, "ms") / 4 / share(dp)
                act = slope(entry, t, "act") / tp * world / bsz
                param_by_tp[t][tp], act_by_tp[t][tp] = par, act
                param_size[t] = max(param_size[t], par * tp)
        # activation per sample under checkpointing
        for t in range(T):
            best = -1.0
            for tp in tps:
                entry = cfg.get(self._strategy(1, tp, world, ckpt=True))
                if entry is not None:
                    best = max(best, slope(entry, t, "act") / tp * world / bsz)
            act_by_tp[t]["checkpoint"] = best

        # what is left on the first / last stage after the layers are accounted for: embeddings, head, norm, loss
        other = {name: {"model_states": {}, "activation": {}} for name in ("off", "on_first", "on_last")}

        def keep_min(table, key, value):
            table[key] = min(table.get(key, INF_MB), max(value, 0))

        pp = 1
        while pp <= world:
            for tp in tps:
                if pp * tp > world or tp not in param_by_tp[0]:
                    continue
                dp = world // pp // tp
                for vtp in ((False,) if tp == 1 else (False, True)):
                    entry = cfg.get(self._strategy(pp, tp, world, vtp=vtp))
                    if entry is None:
                        continue
                    n_layers = pp if pp > 1 else base[0]
                    layernums = [n_layers] * T if pp > 1 else base
                    ms_cost = [param_by_tp[t][tp] * 4 for t in range(T)]
                    act_cost = [act_by_tp[t][tp] for t in range(T)]
                    vocab_div = tp if vtp else 1
                    for stage_rank, stage, names in ((0, 0, ("off", "on_first")), (world - 1, pp - 1, ("off", "on_last"))):
                        name = names[0] if pp == 1 else names[1]
                        if pp == 1 and stage_rank != 0:
                            continue
                        ms = entry[raw_key(layernums, bsz, tag, stage_rank, "ms")]
                        layers_ms = stage_cost(pp, n_layers, ms_cost, stage)
                        # embedding / head states are sharded over the stage's ranks (over its data-parallel ranks only
                        # when the vocabulary is tensor-parallel)
                        other_ms = (ms - layers_ms * share(dp)) / share(world // pp // vocab_div)
                        peak = max(entry[raw_key(layernums, bsz, tag, stage_rank, "act_peak")],
                                   entry[raw_key(layernums, bsz, tag, stage_rank, "act")])
                        layers_act = stage_cost(pp, n_layers, act_cost, stage) * (bsz / dp)
                        other_act = (peak - layers_act) / (bsz / world * pp * vocab_div)
                        key = tp if vtp else 1
                        keep_min(other[name]["model_states"], key, other_ms)
                        keep_min(other[name]["activation"], key, other_act)
            pp *= 2

        if a.sequence_parallel:      # degrees that were not profiled: halve the next smaller one
            for tp in (2, 4, 8):
                if tp not in act_by_tp[0] and tp // 2 in act_by_tp[0]:
                    act_by_tp[0][tp] = act_by_tp[0][tp // 2] / 2
                for table in other.values():
                    for kind in ("model_states", "activation"):
                        if tp not in table[kind] and tp // 2 in table[kind]:
                            table[kind][tp] = table[kind][tp // 2] / 2
        else:
            # without sequence parallelism nothing guarantees that embedding / head memory shrinks with the degree
            # (a patch embedding or a classifier head is replicated): un-profiled degrees of the "other" tables take
            # the next smaller degree's figure, an upper bound, so that the search can price those degrees at all
            for tp in (2, 4, 8):
                for table in other.values():
                    for kind in ("model_states", "activation"):
                        if tp not in table[kind] and tp // 2 in table[kind]:
                            table[kind][tp] = table[kind][tp // 2]

        suffix = "_sp" if a.sequence_parallel else ""
        for t in range(T):
            cfg.setdefault("layertype_%d%s" % (t, suffix), {})[str(seq[t])] = {
                "parameter_size": param_size[t], "tp_activation_per_bsz_dict": act_by_tp[t]}
        for name, table in other.items():
            cfg.setdefault("other_memory_pp_%s%s" % (name, suffix), {})[tag[3:]] = copy.deepcopy(table)
