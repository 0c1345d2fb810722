"""Learning-rate schedule and the optimizer facade used by the training programs.

Reference: ``get_optimizer_and_param_scheduler`` (galvatron/core/runtime/utils.py:137-167: apex FusedAdam + Megatron's
OptimizerParamScheduler). The optimizer itself is the fused sharded AdamW inside ``parallel/zero.py``; this module
supplies the schedule (constant / linear / cosine / inverse-square-root with linear warm-up) and state round-trips.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass

from .loss_scaler import build_loss_scaler


@dataclass
class ParamScheduler:
    max_lr: float = 1e-4
    min_lr: float = 0.0
    warmup_steps: int = 0
    decay_steps: int = 0
    decay_style: str = "constant"
    num_steps: int = 0

    def get_lr(self) -> float:
        s = self.num_steps
        if self.warmup_steps > 0 and s <= self.warmup_steps:
            return self.max_lr * s / self.warmup_steps
        if self.decay_style == "constant" or self.decay_steps <= 0:
            return self.max_lr
        if s > self.decay_steps:
            return self.min_lr
        if self.decay_style == "inverse-square-root":
            w = max(self.warmup_steps, 1)
            return max(self.min_lr, self.max_lr * w ** 0.5 / max(s, 1) ** 0.5)
        ratio = (s - self.warmup_steps) / max(self.decay_steps - self.warmup_steps, 1)
        if self.decay_style == "linear":
            coeff = 1.0 - ratio
        elif self.decay_style == "cosine":
            coeff = 0.5 * (math.cos(math.pi * ratio) + 1.0)
        else:
            raise ValueError("unknown decay style %r" % self.decay_style)
        return self.min_lr + coeff * (self.max_lr - self.min_lr)

    def step(self, increment: int = 1) -> float:
        self.num_steps += increment
        return self.get_lr()

    def state_dict(self) -> dict:
        return dict(vars(self))

    def load_state_dict(self, sd: dict) -> None:
        for k, v in sd.items():
            if hasattr(self, k):
                setattr(self, k, v)


class Optimizer:
    """``step()`` / ``zero_grad()`` over a GalvatronModel's ZeRO engine with the schedule applied."""

    def __init__(self, model, args):
        self.model, self.args = model, args
        iters = getattr(args, "train_iters", None) or 0
        bsz = getattr(args, "global_train_batch_size", 1)
        decay = (getattr(args, "lr_decay_iters", None) or iters) * bsz
        frac = getattr(args, "lr_warmup_fraction", None)
        warm = int(frac * decay) if frac else getattr(args, "lr_warmup_iters", 0) * bsz
        self.scheduler = ParamScheduler(max_lr=args.lr, min_lr=getattr(args, "min_lr", 0.0), warmup_steps=warm, decay_steps=decay,
                                        decay_style=getattr(args, "lr_decay_style", "constant") if iters else "constant")
        self.last_grad_norm = None
        self.scaler = build_loss_scaler(args)
        self.skipped_last_step = False
        if self.scaler is not None:
            model.set_loss_scale(self.scaler.scale)

    @property
    def loss_scale(self) -> float:
        return self.scaler.scale if self.scaler is not None else 1.0

    @property
    def lr(self) -> float:
        return self.scheduler.get_lr() if self.scheduler.num_steps else self.scheduler.max_lr

    @property
    def param_groups(self):
        """One group carrying the current learning rate, for loops written as ``for g in optimizer.param_groups: lr = g["lr"]``
        (reference: models/llama_hf/train_dist.py:88-89)."""
        return [{"lr": self.lr}]

    def step(self):
        a = self.args
        lr = self.lr
        self.last_grad_norm = self.model.optimizer_step(
            lr, beta1=getattr(a, "adam_beta1", 0.9), beta2=getattr(a, "adam_beta2", 0.999), eps=getattr(a, "adam_eps", 1e-8),
            weight_decay=getattr(a, "adam_weight_decay", getattr(a, "weight_decay", 0.01)), max_grad_norm=getattr(a, "clip_grad", 0.0),
            loss_scale=self.loss_scale)
        if self.scaler is not None:
            self.skipped_last_step = bool(self.model.engine.last_step_skipped)
            self.scaler.update(self.skipped_last_step)
            self.model.set_loss_scale(self.scaler.scale)      # the next iteration's losses
        return self.last_grad_norm

    def zero_grad(self):
        self.model.zero_grad()


def get_optimizer_and_param_scheduler(model, args):
    opt = Optimizer(model, args)
    if getattr(args, "load", None) and getattr(args, "distributed_checkpoint", False):
        path = os.path.join(args.load, "iter_%d" % getattr(args, "load_iteration", 0), "opt_param_scheduler.json")
        if os.path.exists(path):
            sd = json.load(open(path))
            opt.scheduler.load_state_dict(sd)
            if opt.scaler is not None and "loss_scaler" in sd:
                opt.scaler.load_state_dict(sd["loss_scaler"])
                model.set_loss_scale(opt.scaler.scale)
    return opt, opt.scheduler


def clip_grad_norm(model, max_norm: float):
    """Global gradient norm (the clip itself is folded into the fused AdamW step through a device-side coefficient)."""
    return model.engine.grad_norm()
