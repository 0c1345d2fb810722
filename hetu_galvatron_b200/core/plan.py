"""The hybrid-parallel plan: per-layer strategy lists + global knobs, convertible from / to the reference's
strategy JSON and its GLOBAL command-line mode.

Reference behaviour reproduced: GLOBAL mode builds uniform per-layer lists from ``--pp_deg --global_tp_deg
--global_cp_deg --sdp --global_checkpoint --use-ulysses --vocab_tp`` and JSON mode reads the searched plan
(galvatron/core/runtime/hybrid_parallel_config.py:17-110); even pipeline division with the remainder on the last
stage (:85-88); ``chunks = -1`` means ``ceil(local_bsz / 4)`` when pipelining (:351-361); validity checks (:190-217).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional

from ..utils.config_utils import array2str, config2strategy, read_json_config, str2array


@dataclass
class HybridPlan:
    pp_deg: int = 1
    tp_sizes_enc: List[int] = field(default_factory=list)
    tp_consecutive_flags: List[int] = field(default_factory=list)
    cp_sizes_enc: List[int] = field(default_factory=list)
    dp_types_enc: List[int] = field(default_factory=list)      # 1 = ZeRO-3, 0 = default_dp_type
    use_sp: List[int] = field(default_factory=list)            # 1 = the layer's tp size is a Ulysses sp size
    checkpoint_flags_enc: List[int] = field(default_factory=list)
    pp_division: List[int] = field(default_factory=list)
    global_bsz: int = 8
    chunks: int = 1
    pipeline_type: str = "pipedream_flush"
    default_dp_type: str = "ddp"
    vocab_tp: int = 1
    vocab_sp: int = 0
    vocab_cp: int = 1
    embed_sdp: int = 0
    sequence_parallel: bool = False      # Megatron-SP on every tensor-parallel layer

    @property
    def num_layers(self) -> int:
        return len(self.tp_sizes_enc)

    @property
    def pp_ranks_enc(self) -> List[int]:
        out = []
        for stage, n in enumerate(self.pp_division):
            out += [stage] * n
        return out

    # ------------------------------------------------------------------ constructors
    @classmethod
    def from_global(cls, num_layers: int, world_size: int, *, pp_deg=1, global_tp_deg=1, global_cp_deg=1, sdp=0,
                    global_checkpoint=0, use_ulysses=False, vocab_tp=1, vocab_cp=1, chunks=1, global_bsz=8,
                    pipeline_type="pipedream_flush", default_dp_type="ddp", embed_sdp=0, sequence_parallel=False,
                    pp_division: Optional[List[int]] = None) -> "HybridPlan":
        tp = max(global_tp_deg, 1)
        cp = max(global_cp_deg, 1)
        plan = cls(pp_deg=pp_deg, tp_sizes_enc=[tp] * num_layers, tp_consecutive_flags=[1] * num_layers,
                   cp_sizes_enc=[cp] * num_layers, dp_types_enc=[int(sdp)] * num_layers,
                   use_sp=[1 if use_ulysses else 0] * num_layers, checkpoint_flags_enc=[int(global_checkpoint)] * num_layers,
                   global_bsz=global_bsz, chunks=chunks, pipeline_type=pipeline_type, default_dp_type=default_dp_type,
                   vocab_tp=vocab_tp, vocab_sp=1 if use_ulysses else 0, vocab_cp=vocab_cp, embed_sdp=embed_sdp,
                   sequence_parallel=sequence_parallel)
        plan.pp_division = pp_division or even_pp_division(num_layers, pp_deg)
        plan.resolve_chunks(world_size)
        return plan

    @classmethod
    def from_json(cls, config, num_layers: Optional[int] = None, sequence_parallel: bool = False,
                  pipeline_type: str = "pipedream_flush", default_dp_type: str = "ddp", embed_sdp: int = 0) -> "HybridPlan":
        cfg = read_json_config(config) if isinstance(config, str) else dict(config)
        pp, tp, cp, consec, dpt, use_sp, vtp, vsp, vcp = config2strategy(cfg)
        n = len(tp)
        if num_layers is not None and n != num_layers:
            raise ValueError("Layer_num in json config (%d) does not match layer_num in the model (%d)" % (n, num_layers))
        plan = cls(pp_deg=pp, tp_sizes_enc=tp, tp_consecutive_flags=consec, cp_sizes_enc=cp, dp_types_enc=dpt, use_sp=use_sp,
                   checkpoint_flags_enc=str2array(cfg["checkpoint"]) if "checkpoint" in cfg else [0] * n,
                   global_bsz=cfg.get("global_bsz", 8), chunks=cfg.get("chunks", 1),
                   pipeline_type=cfg.get("pipeline_type", pipeline_type),
                   default_dp_type=cfg.get("default_dp_type", default_dp_type), vocab_tp=vtp, vocab_sp=vsp, vocab_cp=vcp,
                   embed_sdp=cfg.get("embed_sdp", embed_sdp),
                   sequence_parallel=bool(cfg.get("sequence_parallel", sequence_parallel)))
        plan.pp_division = str2array(cfg["pp_division"]) if "pp_division" in cfg else even_pp_division(n, pp)
        return plan

    # ------------------------------------------------------------------ output
    def to_json(self) -> dict:
        return {
            "pp_deg": self.pp_deg,
            "tp_sizes_enc": array2str(self.tp_sizes_enc),
            "tp_consecutive_flags": array2str(self.tp_consecutive_flags),
            "dp_types_enc": array2str(self.dp_types_enc),
            "use_sp": array2str(self.use_sp),
            "cp_sizes_enc": array2str(self.cp_sizes_enc),
            "checkpoint": array2str(self.checkpoint_flags_enc),
            "global_bsz": self.global_bsz,
            "chunks": self.chunks,
            "pp_division": array2str(self.pp_division),
            "pipeline_type": self.pipeline_type,
            "default_dp_type": self.default_dp_type,
            "vtp": self.vocab_tp,
            "vsp": self.vocab_sp,
            "vcp": self.vocab_cp,
            "embed_sdp": self.embed_sdp,
        }

    def as_runtime_dict(self) -> dict:
        """The dict the reference stores next to a distributed checkpoint (hybrid_parallel_configs.json)."""
        return {
            "pp_deg": self.pp_deg, "tp_sizes_enc": self.tp_sizes_enc, "tp_consecutive_flags": self.tp_consecutive_flags,
            "cp_sizes_enc": self.cp_sizes_enc, "dp_types_enc": self.dp_types_enc,
            "checkpoint_flags_enc": self.checkpoint_flags_enc, "pp_ranks_enc": self.pp_ranks_enc,
            "pp_division": self.pp_division, "use_sp": self.use_sp, "vocab_tp": self.vocab_tp,
            "vocab_sp": self.vocab_sp, "vocab_cp": self.vocab_cp, "default_dp_type": self.default_dp_type,
            "global_train_batch_size": self.global_bsz,
        }

    # ------------------------------------------------------------------ checks
    def resolve_chunks(self, world_size: int) -> int:
        if self.chunks == -1:
            self.chunks = 1
            if self.pp_deg > 1:
                max_dp = world_size // self.pp_deg // max(min(self.tp_sizes_enc + [self.vocab_tp]), 1)
                local_bsz = self.global_bsz // max(max_dp, 1)
                self.chunks = max(int(math.ceil(local_bsz / 4)), 1)
        return self.chunks

    def validate(self, world_size: int, num_heads: Optional[int] = None, num_kv_heads: Optional[int] = None) -> None:
        n = self.num_layers
        for name in ("tp_consecutive_flags", "cp_sizes_enc", "dp_types_enc", "use_sp", "checkpoint_flags_enc"):
            assert len(getattr(self, name)) == n, "%s must have one entry per layer" % name
        assert world_size % self.pp_deg == 0, "world size must be divisible by pp_deg"
        stage = world_size // self.pp_deg
        assert sum(self.pp_division) == n and len(self.pp_division) == self.pp_deg, "pp_division must cover all layers"
        for i, (tp, cp) in enumerate(zip(self.tp_sizes_enc, self.cp_sizes_enc)):
            assert tp >= 1 and cp >= 1 and stage % (tp * cp) == 0, "layer %d: tp*cp must divide the stage size" % i
            assert tp & (tp - 1) == 0, "tp sizes must be powers of two"
            if num_heads is not None and self.use_sp[i]:
                assert num_heads % tp == 0, "Ulysses needs heads divisible by the sp size"
            if num_kv_heads is not None and not self.use_sp[i]:
                assert num_kv_heads % tp == 0, \
                    "layer %d: tensor parallelism needs the KV-head count (%d) divisible by the tp degree (%d)" % (i, num_kv_heads, tp)
        assert stage % (self.vocab_tp * self.vocab_cp) == 0
        min_tp = min(min(self.tp_sizes_enc), self.vocab_tp) if n else self.vocab_tp
        min_cp = min(min(self.cp_sizes_enc), self.vocab_cp) if n else self.vocab_cp
        assert self.global_bsz % (world_size // self.pp_deg // min_tp // min_cp) == 0, \
            "global_train_batch_size should be multiple of world_size//pp_deg//min_tp//min_cp!"
        assert self.global_bsz % self.chunks == 0, "global batch must divide into the micro-batches"
        assert self.pipeline_type in ("gpipe", "pipedream_flush")
        assert self.default_dp_type in ("ddp", "zero2", "zero3")

    def layer_dp_type(self, i: int) -> str:
        return "zero3" if self.dp_types_enc[i] else self.default_dp_type

    def describe(self) -> str:
        lines = ["======================== Galvatron Parallel Config =============================",
                 "   global_batch_size: %d, chunks: %d, pp_deg: %d" % (self.global_bsz, self.chunks, self.pp_deg),
                 "   pipeline_type: %s, default_dp_type: %s%s" % (self.pipeline_type, self.default_dp_type,
                                                                 ", embed_sdp: 1" if self.embed_sdp else "")]
        for k in ("tp_sizes_enc", "cp_sizes_enc", "dp_types_enc", "use_sp", "checkpoint_flags_enc", "pp_division"):
            lines.append("   %s: %s" % (k, array2str(getattr(self, k))))
        lines.append("   vocab_tp: %d, vocab_sp: %d, vocab_cp: %d" % (self.vocab_tp, self.vocab_sp, self.vocab_cp))
        lines.append("================================================================================")
        return "\n".join(lines)


def even_pp_division(num_layers: int, pp_deg: int) -> List[int]:
    avg = num_layers // pp_deg
    return [avg] * (pp_deg - 1) + [num_layers - avg * (pp_deg - 1)]
