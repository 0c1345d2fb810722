"""Pipeline engine: stage execution, micro-batching and the three schedules of the reference
(galvatron/core/runtime/pipeline/pipeline.py): gradient accumulation without a pipeline (:295-373),
GPipe (:718-883) and 1F1B-flush / PipeDream-flush (:375-701).

Stage-to-stage activations travel as NCCL (or gloo) point-to-point messages between ranks with the same
index inside their stage; the tensor keeps the layout of the sending module and the first module of the
receiving stage redistributes it if its own layout differs. Every exchange between two neighbouring stages
posts its sends and receives together as one batched group and waits for the group on the stream (no
``cuda.synchronize``; the reference waits and synchronises the device after every message,
pipeline.py:1125-1127,1244), so the two directions between a pair of stages cannot block each other.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist
import torch.nn as nn

from ..models.transformer import BatchCtx
from .mesh import Mesh
from .reshard import Layout, redistribute
from .zero import ZeroEngine


class StageModule(nn.Module):
    """The modules of one pipeline stage, run in order with a relayout where adjacent layouts differ
    (reference: PipeSequential pipeline.py:1581-1593 + Module_with_relocation parallel.py:279-313)."""

    def __init__(self, blocks: Sequence[nn.Module], layouts: Sequence[Layout], kinds: Sequence[str], mesh: Mesh,
                 in_layout: Optional[Layout], impl: str = "nccl"):
        super().__init__()
        self.blocks = nn.ModuleList(blocks)
        self.layouts = list(layouts)
        self.kinds = list(kinds)
        self.mesh = mesh
        self.in_layout = in_layout      # layout of the tensor received from the previous stage (None on stage 0)
        self.impl = impl

    def forward(self, x, ctx: BatchCtx, stage_batch: int):
        cur = self.in_layout
        for blk, lay, kind in zip(self.blocks, self.layouts, self.kinds):
            if kind != "embed" and cur is not None and cur != lay and torch.is_tensor(x):
                seq = ctx.extra.get("act_seq") or x.shape[0] // ctx.batch * cur.seq_parts()
                x, ctx.batch = redistribute(x, ctx.batch, cur, lay, self.mesh, stage_batch, seq, self.impl)
            elif kind != "embed" and isinstance(x, (tuple, list)) and cur is not None and cur != lay:
                outs = []
                nb = ctx.batch
                for t in x:
                    t2, nb = redistribute(t, ctx.batch, cur, lay, self.mesh, stage_batch, t.shape[0] // ctx.batch * cur.seq_parts(), self.impl)
                    outs.append(t2)
                x, ctx.batch = tuple(outs), nb
            x = blk(x, ctx)
            cur = lay
        return x


class PipelineParallel:
    def __init__(self, stage: StageModule, mesh: Mesh, engine: ZeroEngine, *, chunks: int, pipeline_type: str,
                 stage_batch: int, recv_shape_fn: Callable[[int], List[torch.Size]], act_dtype: torch.dtype, device,
                 make_ctx: Callable, loss_scale_by_chunks: bool = True):
        self.stage, self.mesh, self.engine = stage, mesh, engine
        self.chunks, self.pipeline_type = chunks, pipeline_type
        self.stage_batch = stage_batch          # sequences per micro-batch over the whole stage
        self.recv_shape_fn = recv_shape_fn
        self.act_dtype, self.device = act_dtype, device
        self.make_ctx = make_ctx
        self.prev, self.next = mesh.pp_prev_next()
        self.is_first, self.is_last = mesh.stage == 0, mesh.stage == mesh.pp_deg - 1

    # ------------------------------------------------------------------ p2p
    def _exchange(self, send_to: Optional[int], send_tensors, recv_from: Optional[int], recv_shapes):
        """One batched group of point-to-point messages (sends and receives posted together, so the two
        directions between a pair of stages cannot block each other); returns the received tensors."""
        ops, bufs = [], []
        if send_to is not None and send_tensors:
            send_tensors = [t.contiguous() for t in send_tensors]
            ops += [dist.P2POp(dist.isend, t, send_to) for t in send_tensors]
        if recv_from is not None and recv_shapes:
            bufs = [torch.empty(sh, dtype=self.act_dtype, device=self.device) for sh in recv_shapes]
            ops += [dist.P2POp(dist.irecv, b, recv_from) for b in bufs]
        if ops:
            for r in dist.batch_isend_irecv(ops):
                r.wait()
        return bufs

    # ------------------------------------------------------------------ one micro-batch
    def _forward_compute(self, micro, inputs):
        ctx = self.make_ctx(micro)
        if self.is_first:
            x = micro["input"]
        else:
            for t in inputs:
                t.requires_grad_(True)
            x = inputs[0] if len(inputs) == 1 else tuple(inputs)
        out = self.stage(x, ctx, self.stage_batch)
        if self.is_last:
            loss = out / self.chunks
            return [loss], loss.detach() * self.chunks
        return ([out] if torch.is_tensor(out) else list(out)), None

    def _backward_compute(self, inputs, outputs, grads, last_microbatch: bool):
        self.engine.set_last_microbatch(last_microbatch)
        if self.is_last:
            grads = [None] * len(outputs)
        outs = [o for o in outputs if o.requires_grad]
        gs = [g for o, g in zip(outputs, grads) if o.requires_grad]
        if outs:
            torch.autograd.backward(outs, gs)
        self.engine.finalize_backward()
        if self.is_first:
            return []
        return [t.grad if t.grad is not None else torch.zeros_like(t) for t in inputs]

    def _in_shapes(self, micro):
        return self.recv_shape_fn(micro)

    # ------------------------------------------------------------------ schedules
    def forward_backward(self, micro_batches: List[dict], forward_only: bool = False):
        n = len(micro_batches)
        losses = []
        prev = None if self.is_first else self.prev
        nxt = None if self.is_last else self.next

        def fwd(i, inputs):
            outs, l = self._forward_compute(micro_batches[i], inputs)
            if l is not None:
                losses.append(l)
            return outs

        if forward_only:
            with torch.no_grad():
                for i in range(n):
                    inputs = self._exchange(None, None, prev, self._in_shapes(micro_batches[i]) if prev is not None else None)
                    outs = fwd(i, inputs)
                    self._exchange(nxt, [o.detach() for o in outs] if nxt is not None else None, None, None)
            return losses

        if self.mesh.pp_deg == 1:
            for i in range(n):
                outs = fwd(i, [])
                self._backward_compute([], outs, None, i == n - 1)
            return losses

        if self.pipeline_type == "gpipe":
            saved = []
            for i in range(n):
                inputs = self._exchange(None, None, prev, self._in_shapes(micro_batches[i]) if prev is not None else None)
                outs = fwd(i, inputs)
                self._exchange(nxt, [o.detach() for o in outs] if nxt is not None else None, None, None)
                saved.append((inputs, outs))
            for i, (inputs, outs) in enumerate(saved):
                grads = self._exchange(None, None, nxt, [o.shape for o in outs] if nxt is not None else None)
                ig = self._backward_compute(inputs, outs, grads, i == n - 1)
                self._exchange(prev, ig if prev is not None else None, None, None)
            return losses

        # 1F1B-flush
        warm = min(self.mesh.pp_deg - self.mesh.stage - 1, n)
        steady = n - warm
        fifo = []
        fi = 0
        for _ in range(warm):
            inputs = self._exchange(None, None, prev, self._in_shapes(micro_batches[fi]) if prev is not None else None)
            outs = fwd(fi, inputs)
            self._exchange(nxt, [o.detach() for o in outs] if nxt is not None else None, None, None)
            fifo.append((inputs, outs))
            fi += 1
        inputs = None
        if steady > 0:
            inputs = self._exchange(None, None, prev, self._in_shapes(micro_batches[fi]) if prev is not None else None)
        done = 0
        for k in range(steady):
            outs = fwd(fi, inputs)
            fifo.append((inputs, outs))
            fi += 1
            # send this forward, receive the gradient of the oldest in-flight micro-batch, in one group
            b_in, b_out = fifo.pop(0)
            grads = self._exchange(nxt, [o.detach() for o in outs] if nxt is not None else None,
                                   nxt, [o.shape for o in b_out] if nxt is not None else None)
            done += 1
            ig = self._backward_compute(b_in, b_out, grads, done == n)
            if k == steady - 1:
                self._exchange(prev, ig if prev is not None else None, None, None)
                inputs = None
            else:
                inputs = self._exchange(prev, ig if prev is not None else None,
                                        prev, self._in_shapes(micro_batches[fi]) if prev is not None else None)
        while fifo:
            b_in, b_out = fifo.pop(0)
            grads = self._exchange(None, None, nxt, [o.shape for o in b_out] if nxt is not None else None)
            done += 1
            ig = self._backward_compute(b_in, b_out, grads, done == n)
            self._exchange(prev, ig if prev is not None else None, None, None)
        return losses
