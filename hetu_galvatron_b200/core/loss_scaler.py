"""Loss scaling for fp16 training.

The reference runs fp16 through FSDP's ``MixedPrecision(param_dtype=torch.float16)``
(galvatron/core/runtime/parallel.py:116-122) and leaves loss scaling to the vendored Megatron optimizer
(galvatron/site_package/megatron/core/optimizer/grad_scaler.py: constant and dynamic scalers); its own trainer
never wires one in. Here the scaler belongs to the optimizer façade: the pipeline engine multiplies each
micro-batch loss by the scale, the ZeRO engine divides it out inside the AdamW kernel (through the same device-side
coefficient that carries the gradient clip), and a step whose global gradient norm is not finite is skipped on every
rank alike (the norm is already summed over the whole job, so all ranks see the same value).

bf16 and fp32 runs keep scale 1 and pay nothing for it.
"""
from __future__ import annotations

from dataclasses import dataclass


class ConstantLossScaler:
    """A fixed scale; overflowing steps are still skipped."""

    dynamic = False

    def __init__(self, scale: float = 1.0):
        assert scale > 0
        self.scale = float(scale)
        self.skipped = 0

    def update(self, found_inf: bool) -> None:
        self.skipped += int(bool(found_inf))

    def state_dict(self) -> dict:
        return {"scale": self.scale, "skipped": self.skipped}

    def load_state_dict(self, sd: dict) -> None:
        self.scale = float(sd.get("scale", self.scale))
        self.skipped = int(sd.get("skipped", 0))


@dataclass
class DynamicLossScaler:
    """Scale that backs off after overflows and grows after a run of clean steps.

    ``hysteresis`` overflowing steps (not necessarily consecutive; the budget refills when the scale grows) are
    tolerated before the scale is multiplied by ``backoff_factor``; after ``growth_interval`` consecutive clean steps
    it is multiplied by ``growth_factor``. Every overflowing step is skipped whether or not it changes the scale.
    """

    scale: float = 2.0 ** 16
    min_scale: float = 1.0
    growth_factor: float = 2.0
    backoff_factor: float = 0.5
    growth_interval: int = 1000
    hysteresis: int = 2

    dynamic = True

    def __post_init__(self):
        assert self.scale > 0 and self.min_scale > 0
        assert self.growth_factor > 1.0 and 0.0 < self.backoff_factor < 1.0
        assert self.growth_interval > 0 and self.hysteresis > 0
        self.scale = float(self.scale)
        self._clean = 0
        self._budget = self.hysteresis
        self.skipped = 0

    def update(self, found_inf: bool) -> None:
        if found_inf:
            self.skipped += 1
            self._clean = 0
            self._budget -= 1
            if self._budget <= 0:
                self.scale = max(self.scale * self.backoff_factor, self.min_scale)
            return
        self._clean += 1
        if self._clean % self.growth_interval == 0:
            self._budget = self.hysteresis
            self.scale *= self.growth_factor

    def state_dict(self) -> dict:
        return {"scale": self.scale, "clean": self._clean, "budget": self._budget, "skipped": self.skipped}

    def load_state_dict(self, sd: dict) -> None:
        self.scale = float(sd.get("scale", self.scale))
        self._clean = int(sd.get("clean", 0))
        self._budget = int(sd.get("budget", self.hysteresis))
        self.skipped = int(sd.get("skipped", 0))


def build_loss_scaler(args):
    """Scaler for a run: None unless the run computes in fp16 (or a constant ``--loss_scale`` is asked for)."""
    fixed = getattr(args, "loss_scale", None)
    if fixed:
        return ConstantLossScaler(fixed)
    if getattr(args, "mixed_precision", "bf16") != "fp16":
        return None
    return DynamicLossScaler(scale=getattr(args, "initial_loss_scale", 2.0 ** 16), min_scale=getattr(args, "min_loss_scale", 1.0),
                             growth_interval=getattr(args, "loss_scale_window", 1000), hysteresis=getattr(args, "hysteresis", 2))
