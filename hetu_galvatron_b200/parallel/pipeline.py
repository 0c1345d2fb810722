"""Pipeline engine: stage execution, micro-batching and the three schedules of the reference
(galvatron/core/runtime/pipeline/pipeline.py): gradient accumulation without a pipeline (:295-373),
GPipe (:718-883) and 1F1B-flush / PipeDream-flush (:375-701).

Stage-to-stage activations travel as NCCL (or gloo) point-to-point messages between ranks with the same
index inside their stage; the tensor keeps the layout of the sending module and the first module of the
receiving stage redistributes it if its own layout differs.

The reference waits for every message and then synchronises the whole device (pipeline.py:1125-1127,1244). Here the
messages are posted on a communication stream of their own, ordered against the compute stream with events only:
posting returns at once, the compute stream waits for a message where its data is first used, a forward output is on
the wire while the next micro-batch computes, and the receive of the next forward input is posted before the
backward pass that precedes it (one micro-batch ahead), so the transfer hides behind that backward pass. Receive
buffers come from a per-shape pool and go back to it after the backward pass that consumed them.
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


class _Pending:
    """A posted group of point-to-point messages. ``wait`` orders the CURRENT stream after the group (CUDA) or
    blocks until the requests finished (CPU ranks) and returns the receive buffers."""

    def __init__(self, bufs, reqs=(), event=None):
        self.bufs, self.reqs, self.event = bufs, list(reqs), event

    def wait(self):
        if self.event is not None:
            torch.cuda.current_stream().wait_event(self.event)
            self.event = None
        for r in self.reqs:
            r.wait()
        self.reqs = []
        return self.bufs


class PipelineParallel:
    def __init__(self, stage: StageModule, mesh: Mesh, engine: ZeroEngine, *, chunks: int, pipeline_type: str,
                 stage_batch: int, recv_shape_fn: Callable[[int], List[torch.Size]], act_dtype: torch.dtype, device,
                 make_ctx: Callable, loss_scale_by_chunks: bool = True):
        self.stage, self.mesh, self.engine = stage, mesh, engine
        self.chunks, self.pipeline_type = chunks, pipeline_type
        self.loss_scale = 1.0            # set per iteration by the optimizer façade's loss scaler (fp16 runs)
        self.stage_batch = stage_batch          # sequences per micro-batch over the whole stage
        self.recv_shape_fn = recv_shape_fn
        self.act_dtype, self.device = act_dtype, device
        self.make_ctx = make_ctx
        self.prev, self.next = mesh.pp_prev_next()
        self.is_first, self.is_last = mesh.stage == 0, mesh.stage == mesh.pp_deg - 1
        cuda = torch.device(device).type == "cuda" and mesh.pp_deg > 1
        self.comm_stream = torch.cuda.Stream(device=device) if cuda else None
        self._pool = {}                 # (shape, dtype) -> free receive buffers
        self._inflight = []
        self._connected = False         # GPU stages: neighbour connections established (see _connect_neighbours)

    # ------------------------------------------------------------------ p2p
    def _recv_buffer(self, shape) -> torch.Tensor:
        free = self._pool.get((tuple(shape), self.act_dtype))
        if free:
            return free.pop()
        return torch.empty(shape, dtype=self.act_dtype, device=self.device)

    def _release(self, tensors) -> None:
        """Receive buffers whose consumer has been issued go back to the pool (the next receive into them is ordered
        after the compute stream's current position, so no copy can land before the consumer has run)."""
        for t in tensors or ():
            if torch.is_tensor(t) and getattr(t, "_gv_pooled", False):
                t.grad = None
                if t.requires_grad:
                    t.requires_grad_(False)
                self._pool.setdefault((tuple(t.shape), t.dtype), []).append(t)

    def _post(self, send_to: Optional[int], send_tensors, recv_from: Optional[int], recv_shapes) -> _Pending:
        """Post one batched group of point-to-point messages (sends and receives of the group progress together, so
        the two directions between a pair of stages cannot block each other) without waiting for it."""
        ops, bufs = [], []
        if send_to is not None and send_tensors:
            send_tensors = [t.contiguous() for t in send_tensors]
            ops += [dist.P2POp(dist.isend, t, send_to) for t in send_tensors]
        else:
            send_tensors = []
        if recv_from is not None and recv_shapes:
            bufs = [self._recv_buffer(sh) for sh in recv_shapes]
            for b in bufs:
                b._gv_pooled = True
            ops += [dist.P2POp(dist.irecv, b, recv_from) for b in bufs]
        if not ops:
            return _Pending(bufs)
        if self.comm_stream is None:
            pending = _Pending(bufs, dist.batch_isend_irecv(ops))
            if send_tensors:
                self._inflight.append((pending, send_tensors))     # CPU ranks: sends nobody waits for are drained at the end
            return pending
        cs = self.comm_stream
        cs.wait_stream(torch.cuda.current_stream())     # what is sent was produced, what is overwritten was consumed there
        with torch.cuda.stream(cs):
            for r in dist.batch_isend_irecv(ops):
                r.wait()                                # orders the communication stream only
            event = cs.record_event()
        for t in send_tensors:
            t.record_stream(cs)
        return _Pending(bufs, (), event)

    def _connect_neighbours(self, micro_batches) -> None:
        """Before the first schedule on GPUs: exchange one dummy message of the largest activation size with each
        neighbour, in both directions, and wait for it.

        The library sets a point-to-point connection up on first use, and that set-up blocks the HOST until the peer
        reaches its matching call. Inside the schedule this can close a cycle: a stage blocks in the set-up of the
        gradient direction while the message grouped with it (the next activation) is not yet on its way, the next
        stage's receive for that activation, posted one micro-batch ahead, stays pending on its GPU, and a first-time
        kernel load there (which may synchronise the device) waits for that receive, so the gradient whose send would
        complete the set-up is never launched. With every direction connected up front, at the real message size,
        posting a message never blocks the host and the cycle cannot form."""
        self._connected = True
        if getattr(self, "comm_stream", None) is None:
            return
        n_in = 0
        if not self.is_first and micro_batches:
            for sh in self._in_shapes(micro_batches[0]):
                m = 1
                for d in sh:
                    m *= int(d)
                n_in = max(n_in, m)
        size = torch.tensor([n_in], dtype=torch.int64, device=self.device)
        dist.all_reduce(size, op=dist.ReduceOp.MAX)                       # every rank of the job runs the schedule
        n = max(int(size.item()), 1)
        ops, keep = [], []
        for peer in (self.next if not self.is_last else None, self.prev if not self.is_first else None):
            if peer is None:
                continue
            out, inp = torch.zeros(n, dtype=self.act_dtype, device=self.device), torch.empty(n, dtype=self.act_dtype, device=self.device)
            keep += [out, inp]
            ops += [dist.P2POp(dist.isend, out, peer), dist.P2POp(dist.irecv, inp, peer)]
        if ops:
            for r in dist.batch_isend_irecv(ops):
                r.wait()
        torch.cuda.synchronize(self.device)

    def _exchange(self, send_to: Optional[int], send_tensors, recv_from: Optional[int], recv_shapes):
        """Post a group and make the compute stream wait for it right away (the data is needed next)."""
        return self._post(send_to, send_tensors, recv_from, recv_shapes).wait()

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
            # the loss scale (fp16 runs) multiplies what is differentiated, never what is reported
            loss = out / self.chunks if self.loss_scale == 1.0 else out * (self.loss_scale / self.chunks)
            return [loss], out.detach()
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
        self._release(grads)
        if self.is_first:
            return []
        ig = [t.grad if t.grad is not None else torch.zeros_like(t) for t in inputs]
        self._release(inputs)
        return ig

    def _in_shapes(self, micro):
        return self.recv_shape_fn(micro)

    # ------------------------------------------------------------------ schedules
    def forward_backward(self, micro_batches: List[dict], forward_only: bool = False):
        if not getattr(self, "_connected", False):
            self._connect_neighbours(micro_batches)
        try:
            return self._run_schedule(micro_batches, forward_only)
        finally:
            for pending, _ in self._inflight:
                pending.wait()
            self._inflight = []

    def _run_schedule(self, micro_batches: List[dict], forward_only: bool = False):
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
                    self._post(nxt, [o.detach() for o in outs] if nxt is not None else None, None, None)
                    self._release(inputs)
            return losses

        if self.mesh.pp_deg == 1:
            for i in range(n):
                outs = fwd(i, [])
                self._backward_compute([], outs, None, i == n - 1)
            return losses

        if self.pipeline_type == "gpipe":
            saved = []
            ahead = self._post(None, None, prev, self._in_shapes(micro_batches[0]) if prev is not None else None)
            for i in range(n):
                inputs = ahead.wait()
                if i + 1 < n:                       # the next input arrives while this micro-batch computes
                    ahead = self._post(None, None, prev, self._in_shapes(micro_batches[i + 1]) if prev is not None else None)
                outs = fwd(i, inputs)
                self._post(nxt, [o.detach() for o in outs] if nxt is not None else None, None, None)
                saved.append((inputs, outs))
            ahead = self._post(None, None, nxt, [o.shape for o in saved[0][1]] if nxt is not None else None)
            for i, (inputs, outs) in enumerate(saved):
                grads = ahead.wait()
                if i + 1 < n:
                    ahead = self._post(None, None, nxt, [o.shape for o in saved[i + 1][1]] if nxt is not None else None)
                ig = self._backward_compute(inputs, outs, grads, i == n - 1)
                self._post(prev, ig if prev is not None else None, None, None)
            return losses

        # 1F1B-flush
        warm = min(self.mesh.pp_deg - self.mesh.stage - 1, n)
        steady = n - warm
        fifo = []
        fi = 0
        in_shapes = (lambda i: self._in_shapes(micro_batches[i])) if prev is not None else (lambda i: None)
        ahead = self._post(None, None, prev, in_shapes(0)) if n > 0 else _Pending([])
        for _ in range(warm):
            inputs = ahead.wait()
            ahead = self._post(None, None, prev, in_shapes(fi + 1)) if fi + 1 < n else _Pending([])
            outs = fwd(fi, inputs)
            self._post(nxt, [o.detach() for o in outs] if nxt is not None else None, None, None)
            fifo.append((inputs, outs))
            fi += 1
        done = 0
        for k in range(steady):
            inputs = ahead.wait()
            outs = fwd(fi, inputs)
            fifo.append((inputs, outs))
            fi += 1
            # send this forward, receive the gradient of the oldest in-flight micro-batch, in one group
            b_in, b_out = fifo.pop(0)
            g_pending = self._post(nxt, [o.detach() for o in outs] if nxt is not None else None,
                                   nxt, [o.shape for o in b_out] if nxt is not None else None)
            # the next forward input is received while the backward pass below runs
            ahead = self._post(None, None, prev, in_shapes(fi)) if fi < n else _Pending([])
            grads = g_pending.wait()
            done += 1
            ig = self._backward_compute(b_in, b_out, grads, done == n)
            self._post(prev, ig if prev is not None else None, None, None)
        g_pending = None
        if fifo:
            g_pending = self._post(None, None, nxt, [o.shape for o in fifo[0][1]] if nxt is not None else None)
        while fifo:
            b_in, b_out = fifo.pop(0)
            grads = g_pending.wait()
            if fifo:
                g_pending = self._post(None, None, nxt, [o.shape for o in fifo[0][1]] if nxt is not None else None)
            done += 1
            ig = self._backward_compute(b_in, b_out, grads, done == n)
            self._post(prev, ig if prev is not None else None, None, None)
        return losses
