"""Activation checkpointing: run a block without saving activations, re-run it in backward.

Own implementation of the reference's per-layer ``checkpoint_wrapper`` (galvatron/core/runtime/parallel.py:229-240).
The recomputation re-runs the block's kernels, including any collectives inside it, and restores the RNG state
so dropout masks repeat."""
from __future__ import annotations

import copy
import dataclasses

import torch


def _snapshot(a):
    """Private copy of a per-micro-batch metadata object (a dataclass such as ``BatchCtx``): the stage runner keeps
    mutating the one it passes along (local batch size after each relayout, labels, positions), and the recomputation
    must see the values the block saw in its first forward, not whatever the last module of the stage left behind."""
    if dataclasses.is_dataclass(a) and not isinstance(a, type):
        c = copy.copy(a)
        for f in dataclasses.fields(c):
            v = getattr(c, f.name)
            if isinstance(v, dict):
                setattr(c, f.name, dict(v))
        return c
    return a


class _CheckpointFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, run_fn, kwargs, *args):
        ctx.run_fn, ctx.kwargs = run_fn, kwargs
        ctx.cpu_rng = torch.get_rng_state()
        ctx.cuda_rng = torch.cuda.get_rng_state() if torch.cuda.is_available() and any(
            torch.is_tensor(a) and a.is_cuda for a in args) else None
        ctx.tensor_idx = [i for i, a in enumerate(args) if torch.is_tensor(a)]
        ctx.other = [None if torch.is_tensor(a) else _snapshot(a) for a in args]
        ctx.save_for_backward(*[args[i] for i in ctx.tensor_idx])
        with torch.no_grad():
            out = run_fn(*args, **kwargs)
        return out

    @staticmethod
    def backward(ctx, *grads):
        saved = ctx.saved_tensors
        args = [_snapshot(a) for a in ctx.other]
        detached = []
        for i, t in zip(ctx.tensor_idx, saved):
            d = t.detach()
            d.requires_grad_(t.requires_grad)
            args[i] = d
            detached.append(d)
        cpu_now = torch.get_rng_state()
        cuda_now = torch.cuda.get_rng_state() if ctx.cuda_rng is not None else None
        torch.set_rng_state(ctx.cpu_rng)
        if ctx.cuda_rng is not None:
            torch.cuda.set_rng_state(ctx.cuda_rng)
        with torch.enable_grad():
            out = ctx.run_fn(*args, **ctx.kwargs)
        torch.set_rng_state(cpu_now)
        if cuda_now is not None:
            torch.cuda.set_rng_state(cuda_now)
        outs = (out,) if torch.is_tensor(out) else tuple(out)
        pairs = [(o, g) for o, g in zip(outs, grads) if torch.is_tensor(o) and o.requires_grad and g is not None]
        if pairs:
            torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        res = [None, None]
        it = iter(detached)
        for i, a in enumerate(ctx.other):
            if i in ctx.tensor_idx:
                d = next(it)
                res.append(d.grad if d.requires_grad else None)
            else:
                res.append(None)
        return tuple(res)


def checkpoint(run_fn, *args, **kwargs):
    """Tensors inside tuple / list arguments (an encoder-decoder block receives (encoder states, decoder states)) are
    passed to the autograd Function one by one, so that each gets its gradient from the recomputation."""
    flat, spec = [], []
    for a in args:
        if isinstance(a, (tuple, list)) and any(torch.is_tensor(t) for t in a):
            spec.append((type(a), len(a)))
            flat.extend(a)
        else:
            spec.append(None)
            flat.append(a)
    if all(s is None for s in spec):
        return _CheckpointFn.apply(run_fn, kwargs, *args)

    def regrouped(*flat_args, **kw):
        it = iter(flat_args)
        rebuilt = [next(it) if s is None else s[0](next(it) for _ in range(s[1])) for s in spec]
        return run_fn(*rebuilt, **kw)

    return _CheckpointFn.apply(regrouped, kwargs, *flat)
