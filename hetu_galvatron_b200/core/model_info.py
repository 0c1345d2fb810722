"""``ModelInfo``: the per-module description the reference asks every model family to provide
(galvatron/core/runtime/hybrid_parallel_config.py:161-187: ``layernums / shapes / dtypes / module_types``, where ``-1``
in a shape stands for the micro-batch size and module types ending in ``enc`` / ``dec`` are the searched layers). Here
it is derived from the family's ``ModuleSpec`` list, so a family never writes it by hand."""
from __future__ import annotations

from typing import List, Sequence

import torch


class ModelInfo:
    def __init__(self, cfg, specs: Sequence, sequence_parallel_degree: int = 1):
        self.cfg, self.specs = cfg, list(specs)
        self._sp = max(int(sequence_parallel_degree), 1)

    def layernums(self) -> List[int]:
        """Number of layers of each layer type, in model order (T5: [encoder, decoder]; Swin: one per stage)."""
        counts: List[int] = []
        last = None
        for s in self.specs:
            if s.layer_index is None:
                continue
            key = (s.module_type, getattr(s, "seq_attr", "seq_length"))
            if key != last:
                counts.append(0)
                last = key
            counts[-1] += 1
        return counts

    def module_types(self) -> List[str]:
        return [s.module_type for s in self.specs]

    def shapes(self) -> List[List[List[int]]]:
        """Per module: the shapes of the tensors it hands to the next module, ``[seq / sp, -1, hidden]`` each."""
        out = []
        for s in self.specs:
            n = max(getattr(s, "num_inputs", 1), 1)
            attrs = getattr(s, "seq_attrs", None) or (getattr(s, "seq_attr", "seq_length"),) * n
            hidden = getattr(s, "hidden_size", self.cfg.hidden_size)
            out.append([[(getattr(self.cfg, a, None) or self.cfg.seq_length) // self._sp, -1, hidden] for a in attrs])
        return out

    def dtypes(self) -> List[List[torch.dtype]]:
        return [[self.cfg.dtype] * max(getattr(s, "num_inputs", 1), 1) for s in self.specs]

    def layer_specs(self):
        return [s for s in self.specs if s.layer_index is not None]
