"""Own data-parallel engine: DDP / ZeRO-1 / ZeRO-2 / ZeRO-3 over flat per-block buckets.

The reference wraps every transformer block in PyTorch FSDP1 and monkey-patches its private hooks
(galvatron/core/runtime/parallel.py:92-213,316-386; pipeline/grad_reduce.py:47-65,177-198;
pipeline/sp_grad_reduce.py:93-132). Here one ``ParamBucket`` per block owns

* a flat compute-dtype parameter buffer (ZeRO-3: only this rank's shard is resident; the full buffer is
  all-gathered before the block's forward and backward and dropped afterwards),
* a flat fp32 ``main_grad`` buffer that the weight-gradient GEMMs accumulate into directly,
* fp32 master weights and Adam moments for this rank's shard, updated by one fused kernel.

``dp_type``: ``ddp`` all-reduces gradients and keeps full optimizer state (FSDP NO_SHARD); ``zero2`` keeps full
parameters but reduce-scatters gradients and shards optimizer state (SHARD_GRAD_OP); ``zero3`` also shards the
parameters (FULL_SHARD). With ``async_grad_reduce`` (the reference's default, runtime/arguments.py:179-185)
gradients are reduced once, after the last micro-batch, so full-size gradients persist during accumulation and
ZeRO-2 behaves like ZeRO-1; without it every micro-batch reduce-scatters into the fp32 gradient shard.

``impl="fused"`` (bf16 parameters on CUDA, group of 2..8 ranks on one NVSwitch box) replaces every NCCL call of the
bucket by this package's own peer-memory kernels (csrc/comm_kernels.cu). The gradient bucket and the parameter
buffer live in a symmetric, peer-mapped allocation from the start, so nothing is staged:

* phase A, on a side stream as soon as the block's backward ends: ``gv_grad_reduce`` announces the bucket, waits
  for the peers, sums this rank's slice over all ranks in fp32 into the persistent fp32 gradient shard (writing
  the sum back to everyone for ``ddp``) and announces that it is done reading;
* phase B, after the global gradient norm: ``gv_adamw_push`` updates the fp32 shard and stores the new bf16
  parameters straight into every rank's parameter buffer (ZeRO-2) or into this rank's shard (ZeRO-3), then
  announces the bucket's parameter epoch; the next forward waits for that announcement only;
* ZeRO-3 gathers pull the peers' shards with ``gv_allgather_pull`` on a gather stream, one block ahead of use.

A peer announces its gradients only after its last use of the old parameters in the step, so phase B needs no
extra barrier; a bucket is cleared only after every peer announced that it finished reading it.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional

import ctypes
import os

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import _lib
from ..ops import functional as Fn
from ..utils.trace import get_tracer
from .mesh import CommGroup

ALIGN = 8  # elements; keeps every parameter 16-byte aligned in bf16 and 32-byte aligned in fp32

# flag slots of a bucket's own symmetric workspace
SLOT_READY, SLOT_DONE, SLOT_PARAM = 0, 1, 2
# budget of the device-side waits of the fused path: a peer may legitimately be late by a data-loading or
# checkpointing hiccup, so this is far above the default of the activation kernels (the wait still ends by itself)
ZERO_WAIT_MS = int(os.environ.get("GV_ZERO_WAIT_MS", "30000"))

_SIDE_STREAMS = {}


def _side_stream(kind: str, device) -> "torch.cuda.Stream":
    """One reduction/update stream and one gather stream per device, shared by all buckets."""
    key = (kind, torch.device(device).index)
    st = _SIDE_STREAMS.get(key)
    if st is None:
        st = _SIDE_STREAMS[key] = torch.cuda.Stream(device=device)
    return st


class _EventWork:
    """Stands in for a c10d work handle: ``wait`` makes the current stream wait for the recorded event."""

    def __init__(self, event):
        self.event = event

    def wait(self):
        torch.cuda.current_stream().wait_event(self.event)


class _FusedState:
    """Symmetric workspace of one bucket: [ctrl | gradient bucket | parameter buffer (ZeRO-3: this rank's shard)]."""

    def __init__(self, bucket: "ParamBucket"):
        from .symm import SymmWorkspace

        b = bucket
        gsize = torch.empty(0, dtype=b.grad_dtype).element_size()
        self.gbytes = b.numel * gsize
        self.pnumel = b.shard_numel if b.dp_type == "zero3" else b.numel
        self.ws = SymmWorkspace(b.group, 256 + self.gbytes + self.pnumel * 2 + 1024, device=b.device)
        self.ctr_off = self.ws.region("ctrl", 256)
        self.goff = self.ws.region("grad", self.gbytes)
        self.poff = self.ws.region("param", self.pnumel * 2)
        self.grad = self.ws.view(self.goff, (b.numel,), b.grad_dtype)
        self.param = self.ws.view(self.poff, (self.pnumel,), b.dtype)
        self.stream = _side_stream("reduce", b.device)
        self.gather_stream = _side_stream("gather", b.device)
        self.ge = 0                 # gradient epoch: one per reduction
        self.pe = 0                 # parameter epoch: one per update
        self.shard_buf: Optional[torch.Tensor] = None
        self.shard_valid = False    # the fp32 shard holds a partial sum of this step (per-micro-batch reduction)
        self.dirty = False          # peers may still be reading the gradient bucket
        self.param_event = None
        self.reduce_event = None

    @property
    def peers(self):
        return ctypes.byref(self.ws.peers)



def _align(n: int, a: int) -> int:
    return (n + a - 1) // a * a


class ParamBucket:
    def __init__(self, name: str, params: Iterable[nn.Parameter], group: Optional[CommGroup], dp_type: str = "ddp",
                 grad_dtype: torch.dtype = torch.float32, tp_group: Optional[CommGroup] = None,
                 reduce_dtype: Optional[torch.dtype] = None, impl: str = "nccl"):
        self.name = name
        self.params: List[nn.Parameter] = [p for p in params if p.requires_grad]
        assert dp_type in ("ddp", "zero2", "zero3")
        self.group = group
        self.pg = group.group if group is not None else None
        self.d = group.size if group is not None else 1
        self.grank = group.rank_in_group(dist.get_rank()) if (group is not None and dist.is_initialized() and self.d > 1) else 0
        self.dp_type = dp_type if self.d > 1 else "ddp"
        self.tp_group = tp_group
        self.grad_dtype = grad_dtype
        self.reduce_dtype = reduce_dtype
        self.deferred = False            # reduce only at the end of the step (tied weights shared across stages)
        self.pre_reduce_hooks: list = []
        self.fused: Optional[_FusedState] = None
        self.impl = "nccl"
        self.users = 0                   # blocks that hold parameters of this bucket (tied weights: more than one)
        self._users_done = 0
        if not self.params:
            self.numel = 0
            return
        self._remember_shapes()
        p0 = self.params[0]
        self.device, self.dtype = p0.device, p0.dtype
        self.offsets: List[int] = []
        off = 0
        for p in self.params:
            self.offsets.append(off)
            off += _align(p.numel(), ALIGN)
        self.numel = _align(off, ALIGN * self.d)
        self.shard_numel = self.numel // self.d
        self.lo = self.grank * self.shard_numel if self.dp_type != "ddp" else 0
        self.opt_numel = self.shard_numel if self.dp_type != "ddp" else self.numel

        if impl == "fused" and self._fused_eligible():
            try:
                self.fused = _FusedState(self)
                self.impl = "fused"
            except Exception as exc:          # no peer-mapped memory on this machine: the library collectives still work
                import warnings

                warnings.warn("bucket %s: symmetric memory unavailable (%s: %s); using NCCL collectives"
                              % (name, type(exc).__name__, exc))
                self.fused = None
        if self.fused is not None and self.dp_type != "zero3":
            flat = self.fused.param          # the parameters live in the peer-mapped buffer from the start
        else:
            flat = torch.zeros(self.numel, dtype=self.dtype, device=self.device)
        for p, o in zip(self.params, self.offsets):
            flat[o:o + p._gv_numel].copy_(p.data.reshape(-1))
        # fp32 master copy of this rank's slice
        self.master = flat[self.lo:self.lo + self.opt_numel].float().clone() if self.dtype != torch.float32 else None
        self.exp_avg = torch.zeros(self.opt_numel, dtype=torch.float32, device=self.device)
        self.exp_avg_sq = torch.zeros(self.opt_numel, dtype=torch.float32, device=self.device)
        if self.dp_type == "zero3":
            if self.fused is not None:
                self.param_shard = self.fused.param
                self.param_shard.copy_(flat[self.lo:self.lo + self.shard_numel])
            else:
                self.param_shard = flat[self.lo:self.lo + self.shard_numel].clone()
            self.param_flat = None
            for p in self.params:
                p.data = torch.empty(0, dtype=self.dtype, device=self.device)
            del flat
        else:
            self.param_flat = flat
            self.param_shard = flat[self.lo:self.lo + self.opt_numel]
            self._point_params(flat)
        if self.dtype == torch.float32:
            self.master = self.param_shard  # fp32 training: the parameters are their own master copy
        self.grad_flat: Optional[torch.Tensor] = self.fused.grad if self.fused is not None else None
        self.grad_shard: Optional[torch.Tensor] = None  # fp32 reduced gradient of this rank's slice
        self._works: list = []
        self._param_work = None          # in-flight all-gather of the updated parameters (ZeRO-2, after the step)
        self._prefetch = None            # (work, buffer) of an all-gather started ahead of use (ZeRO-3)
        self.neighbours = (None, None)   # (previous, next) bucket in execution order, set by the engine
        self._unshard_depth = 0
        self.pending_reduce = False
        self.reduced = False
        # parameters whose gradients are partial sums over the TP group (norm weights / post-reduction biases
        # under sequence parallelism) and parameters duplicated over the TP group (for the gradient norm)
        self.sp_params = [i for i, p in enumerate(self.params) if getattr(p, "sequence_parallel", False)]
        self.dup_params = [i for i, p in enumerate(self.params) if getattr(p, "tp_duplicate", False)]
        # copies of a weight whose gradient another pipeline stage already counts in the global norm (tied embedding)
        self.skip_params = [i for i, p in enumerate(self.params) if getattr(p, "norm_skip", False)]

    def _fused_eligible(self) -> bool:
        from . import symm

        return (self.d > 1 and self.device.type == "cuda" and self.dtype == torch.bfloat16
                and self.grad_dtype in (torch.bfloat16, torch.float32) and symm.available(self.group))

    # ------------------------------------------------------------------ parameter views
    def _point_params(self, flat: torch.Tensor) -> None:
        for p, o in zip(self.params, self.offsets):
            p.data = flat[o:o + p._gv_numel].view(p._gv_shape)

    def _remember_shapes(self) -> None:
        for p in self.params:
            p._gv_shape, p._gv_numel = tuple(p.shape), p.numel()

    def _ensure_grad(self) -> None:
        if self.grad_flat is None:
            self.grad_flat = torch.zeros(self.numel, dtype=self.grad_dtype, device=self.device)
        for p, o in zip(self.params, self.offsets):
            p.main_grad = self.grad_flat[o:o + p._gv_numel].view(p._gv_shape)

    # ------------------------------------------------------------------ ZeRO-3 gather / release
    def wait_params(self) -> None:
        """The parameters of this bucket are about to be read: finish the all-gather the optimizer step left running."""
        if self._param_work is not None:
            self._param_work.wait()
            if self.fused is not None:
                # the local part is ordered by the event above; the peers' stores by their announcements
                f = self.fused
                _lib.check(_lib.lib().gv_comm_wait_peers(f.peers, SLOT_PARAM, ctypes.c_uint(f.pe), ZERO_WAIT_MS,
                                                         ctypes.c_void_p(_lib.stream_ptr())), "gv_comm_wait_peers")
            self._param_work = None

    def _start_gather(self):
        full = torch.empty(self.numel, dtype=self.dtype, device=self.device)
        if self.fused is not None:
            # pull every rank's shard out of its peer-mapped buffer; a source is read once it announced the
            # current parameter epoch (its own update of this step has landed)
            f = self.fused
            gs = f.gather_stream
            gs.wait_stream(torch.cuda.current_stream())     # `full` may reuse memory the compute stream still reads
            with torch.cuda.stream(gs):
                _lib.check(_lib.lib().gv_allgather_pull_ex(f.peers, ctypes.c_longlong(f.poff), ctypes.c_void_p(full.data_ptr()),
                                                           ctypes.c_longlong(self.shard_numel), SLOT_PARAM, ctypes.c_uint(f.pe),
                                                           ZERO_WAIT_MS, ctypes.c_void_p(_lib.stream_ptr())), "gv_allgather_pull")
                ev = gs.record_event()
            return _EventWork(ev), full
        work = dist.all_gather_into_tensor(full, self.param_shard, group=self.pg, async_op=True)
        return work, full

    def prefetch(self) -> None:
        """ZeRO-3: start gathering this bucket's parameters now; the next ``unshard`` picks the result up."""
        if self.numel == 0 or self.dp_type != "zero3" or self._unshard_depth > 0 or self._prefetch is not None:
            return
        self._prefetch = self._start_gather()

    def unshard(self, backward: bool = False) -> None:
        if self.numel == 0:
            return
        self.wait_params()
        self._unshard_depth += 1
        if self.dp_type != "zero3" or self._unshard_depth > 1:
            return
        work, full = self._prefetch if self._prefetch is not None else self._start_gather()
        self._prefetch = None
        work.wait()
        self.param_flat = full
        self._point_params(full)
        # overlap the neighbour's gather with this block's compute (next block in forward, previous in backward)
        nxt = self.neighbours[0 if backward else 1]
        if nxt is not None:
            nxt.prefetch()

    def reshard(self) -> None:
        if self.numel == 0:
            return
        self._unshard_depth -= 1
        if self.dp_type != "zero3" or self._unshard_depth > 0:
            return
        self.param_flat = None
        for p in self.params:
            p.data = torch.empty(0, dtype=self.dtype, device=self.device)

    # ------------------------------------------------------------------ gradient reduction
    def _fold_autograd_grads(self) -> None:
        """Parameters used through ordinary PyTorch ops receive ``.grad`` from autograd; move it into main_grad."""
        for p in self.params:
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(p.main_grad.dtype).view(p._gv_shape))
                p.grad = None

    def prepare_backward(self) -> None:
        if self.numel == 0:
            return
        self._ensure_grad()
        self.pending_reduce = True

    def reduce_grads(self, last_microbatch: bool, async_grad_reduce: bool, force: bool = False) -> None:
        """Called when a block's backward for one micro-batch is complete. A bucket that several blocks of the stage
        share (a tied embedding used by the embedding, a decoder embedding and the head) is reduced once, when the last
        of them has finished; ``force`` (end of the backward pass) reduces whatever is still pending."""
        if self.numel == 0 or not self.pending_reduce:
            return
        if self.users > 1 and not force:
            self._users_done += 1
            if self._users_done < self.users:
                return
        self._users_done = 0
        self._fold_autograd_grads()
        if self.deferred:
            return
        self.pending_reduce = False
        if (async_grad_reduce or self.dp_type == "ddp" or self.d == 1) and not last_microbatch:
            return
        # partial-sum gradients under sequence parallelism: sum over the TP group first
        if self.sp_params and self.tp_group is not None and self.tp_group.size > 1 and (last_microbatch or not async_grad_reduce):
            views = [self.grad_flat[self.offsets[i]:self.offsets[i] + self.params[i]._gv_numel] for i in self.sp_params]
            packed = torch.cat(views)
            dist.all_reduce(packed, group=self.tp_group.group)
            o = 0
            for v in views:
                v.copy_(packed[o:o + v.numel()])
                o += v.numel()
        if self.d == 1:
            self.grad_shard = self.grad_flat
            self.reduced = True
            return
        if self.fused is not None:
            self._fused_reduce(async_grad_reduce)
            self.reduced = True
            return
        src = self.grad_flat
        if self.reduce_dtype is not None and self.reduce_dtype != src.dtype:
            src = src.to(self.reduce_dtype)
        if self.dp_type == "ddp":
            w = dist.all_reduce(src, group=self.pg, async_op=True)
            self._works.append((w, "ddp", src))
        else:
            out = torch.empty(self.shard_numel, dtype=src.dtype, device=self.device)
            w = dist.reduce_scatter_tensor(out, src, group=self.pg, async_op=True)
            self._works.append((w, "rs", out))
        self.reduced = True

    def _fused_reduce(self, async_grad_reduce: bool) -> None:
        """Phase A on the reduction stream: the kernel itself announces the bucket and waits for the peers."""
        f = self.fused
        ddp = self.dp_type == "ddp"
        if not ddp and f.shard_buf is None:
            f.shard_buf = torch.empty(self.shard_numel, dtype=torch.float32, device=self.device)
        f.ge += 1
        accumulate = int((not async_grad_reduce) and f.shard_valid and not ddp)
        f.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(f.stream):
            _lib.check(_lib.lib().gv_grad_reduce(
                f.peers, ctypes.c_longlong(f.goff), int(self.grad_dtype == torch.bfloat16),
                ctypes.c_longlong(self.grank * self.shard_numel), ctypes.c_longlong(self.shard_numel),
                ctypes.c_void_p(0 if ddp else f.shard_buf.data_ptr()), accumulate, int(ddp), None,
                ctypes.c_longlong(f.ctr_off), SLOT_READY, SLOT_DONE, ctypes.c_uint(f.ge), ZERO_WAIT_MS, 0,
                ctypes.c_void_p(_lib.stream_ptr())), "gv_grad_reduce")
            f.reduce_event = f.stream.record_event()
        f.shard_valid = True
        f.dirty = True
        self._works.append((None, "fused", None))

    def _fused_clear_grad(self) -> None:
        """Zero the gradient bucket; when peers may still be reading it, only after each announced it is done."""
        f = self.fused
        if f.dirty:
            _lib.check(_lib.lib().gv_wait_zero(f.peers, SLOT_DONE, ctypes.c_uint(f.ge), ctypes.c_void_p(self.grad_flat.data_ptr()),
                                               ctypes.c_longlong(f.gbytes), ZERO_WAIT_MS, ctypes.c_void_p(_lib.stream_ptr())),
                       "gv_wait_zero")
            f.dirty = False
        else:
            self.grad_flat.zero_()

    def finish_reduce(self, async_grad_reduce: bool) -> None:
        if self.fused is not None:
            if not self._works:
                return
            f = self.fused
            torch.cuda.current_stream().wait_event(f.reduce_event)
            if self.dp_type == "ddp":
                # the peers' sums of their slices land in this rank's bucket: wait for their announcements
                _lib.check(_lib.lib().gv_comm_wait_peers(f.peers, SLOT_DONE, ctypes.c_uint(f.ge), ZERO_WAIT_MS,
                                                         ctypes.c_void_p(_lib.stream_ptr())), "gv_comm_wait_peers")
                f.dirty = False
                self.grad_shard = self.grad_flat
            else:
                self.grad_shard = f.shard_buf
                if not async_grad_reduce:
                    self._fused_clear_grad()
            self._works = []
            return
        for w, kind, buf in self._works:
            w.wait()
            if kind == "ddp":
                if buf is not self.grad_flat:
                    self.grad_flat.copy_(buf)
                self.grad_shard = self.grad_flat
            else:
                red = buf if buf.dtype == torch.float32 else buf.float()
                if async_grad_reduce or self.grad_shard is None:
                    self.grad_shard = red
                else:
                    self.grad_shard.add_(red)
                if not async_grad_reduce:
                    self.grad_flat.zero_()
        self._works = []

    def zero_grad(self) -> None:
        if self.numel == 0:
            return
        if self.fused is not None:
            self._fused_clear_grad()
            self.fused.shard_valid = False
        elif self.grad_flat is not None:
            self.grad_flat.zero_()
        if self.dp_type != "ddp" or self.d == 1:
            self.grad_shard = None if self.d > 1 else self.grad_flat
        self.reduced = False

    # ------------------------------------------------------------------ optimizer
    def grad_sumsq(self, out: torch.Tensor, tp_size: int) -> None:
        """Adds this bucket's share of the squared global gradient norm (already divided by d^2) into out[0]."""
        if self.numel == 0 or self.grad_shard is None:
            return
        tmp = torch.zeros(1, dtype=torch.float32, device=self.device)
        Fn.sumsq_accum(self.grad_shard, tmp)

        def part(indices):
            acc = torch.zeros(1, dtype=torch.float32, device=self.device)
            for i in indices:
                a = max(self.offsets[i], self.lo) - self.lo
                b = min(self.offsets[i] + self.params[i]._gv_numel, self.lo + self.opt_numel) - self.lo
                if b > a:
                    Fn.sumsq_accum(self.grad_shard[a:b].contiguous(), acc)
            return acc

        if self.skip_params:
            tmp -= part(self.skip_params)
        dups = [i for i in self.dup_params if i not in self.skip_params]
        if dups and tp_size > 1:
            tmp -= part(dups) * (1.0 - 1.0 / tp_size)
        weight = 1.0 / (self.d * self.d)
        if self.dp_type == "ddp" and self.d > 1:
            weight /= self.d  # every replica holds (and counts) the whole gradient
        out.add_(tmp * weight)

    def step(self, lr, beta1, beta2, eps, weight_decay, step, clip_coef) -> None:
        if self.numel == 0 or self.grad_shard is None:
            return
        self.wait_params()
        if self.fused is not None and self.dp_type != "ddp":
            self._fused_step(lr, beta1, beta2, eps, weight_decay, step, clip_coef)
            return
        low = None if self.dtype == torch.float32 else self.param_shard
        Fn.adamw_step_(self.master, self.exp_avg, self.exp_avg_sq, self.grad_shard, low, lr=lr, beta1=beta1, beta2=beta2,
                       eps=eps, weight_decay=weight_decay, step=step, grad_scale=1.0 / self.d, clip_coef=clip_coef)
        if self.dp_type == "zero2":
            # left running: the first forward that reads these parameters waits for it (wait_params)
            src = self.param_shard if self.param_flat.is_cuda else self.param_shard.clone()
            self._param_work = dist.all_gather_into_tensor(self.param_flat, src, group=self.pg, async_op=True)
        if self.dp_type == "zero3":
            self._prefetch = None            # a gather started before the update holds stale values

    def _fused_step(self, lr, beta1, beta2, eps, weight_decay, step, clip_coef) -> None:
        """Phase B on the reduction stream: AdamW on the shard, new bf16 parameters stored into every rank's buffer
        (ZeRO-2) or into this rank's shard (ZeRO-3); the compute stream carries on and waits per bucket on first use."""
        f = self.fused
        zero3 = self.dp_type == "zero3"
        f.pe += 1
        bc1, bc2 = 1.0 - beta1 ** step, 1.0 - beta2 ** step
        f.stream.wait_stream(torch.cuda.current_stream())
        if clip_coef is not None:
            clip_coef.record_stream(f.stream)
        with torch.cuda.stream(f.stream):
            _lib.check(_lib.lib().gv_adamw_push(
                f.peers, ctypes.c_longlong(f.poff), ctypes.c_longlong(0 if zero3 else self.lo), ctypes.c_longlong(self.shard_numel),
                ctypes.c_void_p(self.master.data_ptr()), ctypes.c_void_p(self.exp_avg.data_ptr()),
                ctypes.c_void_p(self.exp_avg_sq.data_ptr()), ctypes.c_void_p(self.grad_shard.data_ptr()), int(not zero3),
                ctypes.c_float(lr), ctypes.c_float(beta1), ctypes.c_float(beta2), ctypes.c_float(eps),
                ctypes.c_float(weight_decay), ctypes.c_float(bc1), ctypes.c_float(bc2), ctypes.c_float(1.0 / self.d),
                ctypes.c_void_p(_lib.p(clip_coef)), ctypes.c_longlong(f.ctr_off), SLOT_PARAM, ctypes.c_uint(f.pe),
                ctypes.c_void_p(_lib.stream_ptr())), "gv_adamw_push")
            f.param_event = f.stream.record_event()
        if zero3:
            self._prefetch = None            # a gather started before the update holds stale values
            # this rank's own later use of the shard (state_dict, reload) is ordered by the event
            torch.cuda.current_stream().wait_event(f.param_event)
        else:
            self._param_work = _EventWork(f.param_event)

    def sync_peers(self) -> None:
        """After parameters were written outside the optimizer step (construction, checkpoint load): make them
        visible to the peers that will pull or rely on them. Collective over the bucket's group."""
        if self.fused is not None:
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.pg)

    # ------------------------------------------------------------------ state
    def state_dict(self) -> dict:
        self.wait_params()
        return {"master": None if self.master is self.param_shard else self.master, "exp_avg": self.exp_avg,
                "exp_avg_sq": self.exp_avg_sq, "lo": self.lo, "numel": self.numel, "param_shard": self.param_shard}

    def load_state_dict(self, sd: dict) -> None:
        if sd.get("master") is not None and self.master is not self.param_shard:
            self.master.copy_(sd["master"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
        self.wait_params()
        self._prefetch = None
        self.param_shard.copy_(sd["param_shard"])
        if self.dp_type == "zero2":
            dist.all_gather_into_tensor(self.param_flat, self.param_shard.clone(), group=self.pg)
        self.sync_peers()

    def full_optimizer_state(self) -> Dict[str, torch.Tensor]:
        """fp32 master weights and Adam moments of the WHOLE bucket as flat host vectors [numel], whatever the
        sharding (a collective over the bucket's group for ZeRO buckets: every rank of the group must call it)."""
        self.wait_params()

        def whole(x: torch.Tensor) -> torch.Tensor:
            x = x.detach().float().contiguous()
            if self.dp_type == "ddp" or self.d == 1:
                return x.cpu()
            out = torch.empty(self.numel, dtype=torch.float32, device=self.device)
            dist.all_gather_into_tensor(out, x, group=self.pg)
            return out.cpu()

        return {"master": whole(self.master), "exp_avg": whole(self.exp_avg), "exp_avg_sq": whole(self.exp_avg_sq)}

    def load_full_optimizer_state(self, full: Dict[str, torch.Tensor]) -> None:
        """Inverse of ``full_optimizer_state`` under THIS bucket's sharding: keep the local slice of each vector and
        refresh the parameters from the master weights. Call between ``unshard`` and ``reshard``."""
        sl = slice(self.lo, self.lo + self.opt_numel)
        self.exp_avg.copy_(full["exp_avg"][sl])
        self.exp_avg_sq.copy_(full["exp_avg_sq"][sl])
        self._prefetch = None
        assert self.param_flat is not None, "load_full_optimizer_state needs the bucket unsharded"
        self.param_flat.copy_(full["master"].to(device=self.device, dtype=self.dtype))
        self.commit_loaded_params()
        if self.master is not self.param_shard:
            self.master.copy_(full["master"][sl])          # keep the fp32 bits, not the re-rounded bf16 values

    def commit_loaded_params(self) -> None:
        """After new values were written into the (unsharded) parameters: refresh this rank's shard and its
        fp32 master copy from them. Call between ``unshard`` and ``reshard``."""
        if self.numel == 0:
            return
        self._prefetch = None
        assert self.param_flat is not None, "commit_loaded_params needs the bucket unsharded"
        piece = self.param_flat[self.lo:self.lo + self.opt_numel]
        if self.dp_type == "zero3":
            self.param_shard.copy_(piece)
        if self.master is not self.param_shard:
            self.master.copy_(piece.float())
        self.sync_peers()

    def full_params(self) -> Dict[int, torch.Tensor]:
        """Index -> full (unsharded) parameter tensor (a gather for ZeRO-3)."""
        self.unshard()
        out = {i: p.data.clone() for i, p in enumerate(self.params)}
        self.reshard()
        return out


# ---------------------------------------------------------------------- autograd boundary hooks
class _PreBackward(torch.autograd.Function):
    """Identity on the block outputs; its backward runs first in the block's backward pass."""

    @staticmethod
    def forward(ctx, block, *xs):
        ctx.block = block
        return xs if len(xs) > 1 else xs[0]

    @staticmethod
    def backward(ctx, *gs):
        ctx.block._pre_backward()
        return (None,) + gs


class _PostBackward(torch.autograd.Function):
    """Identity on the block inputs; its backward runs last in the block's backward pass."""

    @staticmethod
    def forward(ctx, block, *xs):
        ctx.block = block
        return xs if len(xs) > 1 else xs[0]

    @staticmethod
    def backward(ctx, *gs):
        ctx.block._post_backward()
        return (None,) + gs


class ZeroBlock(nn.Module):
    """One data-parallel unit: a module, its bucket, optional activation checkpointing
    (reference: parallel.py:216-246 checkpoint_wrapper inside the FSDP unit)."""

    def __init__(self, module: nn.Module, bucket: ParamBucket, engine: "ZeroEngine", checkpoint: bool = False,
                 extra_buckets=()):
        super().__init__()
        self.module = module
        self.bucket = bucket
        self.all_buckets = [bucket] + list(extra_buckets)   # a block sharing tied weights spans two buckets
        for b in self.all_buckets:
            b.users += 1
        self.engine = engine
        self.order = engine.register_block()      # position in the stage (forward order)
        self.checkpoint = checkpoint
        self._in_backward = 0

    def _pre_backward(self) -> None:
        self._in_backward += 1
        get_tracer().begin("bwd:" + self.bucket.name, "backward")
        for b in self.all_buckets:
            b.unshard(backward=True)
            b.prepare_backward()
        self.engine._active.add(self)

    def _post_backward(self) -> None:
        if self._in_backward == 0:
            return
        self._in_backward -= 1
        get_tracer().end("bwd:" + self.bucket.name)
        for b in self.all_buckets:
            b.reshard()
            b.reduce_grads(self.engine.last_microbatch, self.engine.async_grad_reduce)
        self.engine._active.discard(self)

    def forward(self, *args, **kwargs):
        for b in self.all_buckets:
            b.unshard()
        grad_mode = torch.is_grad_enabled()
        if grad_mode:
            for b in self.all_buckets:
                if b.numel:
                    b._ensure_grad()
            # every differentiable input tensor -- also inside a tuple / list argument (encoder-decoder blocks take
            # (encoder states, decoder states)) -- goes through the hook that closes the block's backward
            def needs(t):
                return torch.is_tensor(t) and t.requires_grad

            tens = []
            for a in args:
                if needs(a):
                    tens.append(a)
                elif isinstance(a, (tuple, list)):
                    tens.extend(t for t in a if needs(t))
            if tens:
                hooked = _PostBackward.apply(self, *tens)
                hooked = (hooked,) if torch.is_tensor(hooked) else tuple(hooked)
                it = iter(hooked)
                new_args = []
                for a in args:
                    if needs(a):
                        new_args.append(next(it))
                    elif isinstance(a, (tuple, list)):
                        new_args.append(type(a)(next(it) if needs(t) else t for t in a))
                    else:
                        new_args.append(a)
                args = tuple(new_args)
        with get_tracer().span("fwd:" + self.bucket.name, "forward"):
            if self.checkpoint and grad_mode:
                from .checkpointing import checkpoint as ckpt
                out = ckpt(self.module, *args, **kwargs)
            else:
                out = self.module(*args, **kwargs)
        if grad_mode:
            if torch.is_tensor(out):
                if out.requires_grad:
                    out = _PreBackward.apply(self, out)
            else:
                outs = list(out)
                idx = [i for i, o in enumerate(outs) if torch.is_tensor(o) and o.requires_grad]
                if idx:
                    hooked = _PreBackward.apply(self, *[outs[i] for i in idx])
                    hooked = (hooked,) if torch.is_tensor(hooked) else tuple(hooked)
                    for i, h in zip(idx, hooked):
                        outs[i] = h
                out = tuple(outs)
        for b in self.all_buckets:
            b.reshard()
        return out


class ZeroEngine:
    """All buckets of this rank + the fused AdamW step + gradient clipping."""

    def __init__(self, async_grad_reduce: bool = True, world_group=None, tp_size_of_bucket=None):
        self.buckets: List[ParamBucket] = []
        self.async_grad_reduce = async_grad_reduce
        self.last_microbatch = True
        self._active = set()
        self.world_group = world_group
        self.step_count = 0
        self.last_norm = None
        self.last_step_skipped = False

    def add_bucket(self, bucket: ParamBucket) -> ParamBucket:
        if bucket.numel:
            prev = next((b for b in reversed(self.buckets) if b.numel), None)
            bucket.neighbours = (prev, None)
            if prev is not None:
                prev.neighbours = (prev.neighbours[0], bucket)
        self.buckets.append(bucket)
        return bucket

    def sync_symmetric(self) -> None:
        """Call once after all buckets are built: their initial parameters must have landed before a peer pulls them."""
        if any(b.numel and b.fused is not None for b in self.buckets):
            torch.cuda.synchronize()
            dist.barrier()

    @property
    def comm_impl(self) -> str:
        """"fused" when at least one bucket runs on the peer-memory kernels, else "nccl"."""
        return "fused" if any(b.numel and b.fused is not None for b in self.buckets) else "nccl"

    def set_last_microbatch(self, flag: bool) -> None:
        self.last_microbatch = flag

    def register_block(self) -> int:
        self._num_blocks = getattr(self, "_num_blocks", 0) + 1
        return self._num_blocks - 1

    def finalize_backward(self) -> None:
        """After a backward pass: close blocks whose inputs carried no gradient, wait for the reductions. The blocks
        are closed in backward order (never in the iteration order of a set: every rank has to issue the same
        collectives in the same order)."""
        for blk in sorted(self._active, key=lambda b: -b.order):
            blk._post_backward()
        for b in self.buckets:
            if b.numel and b.pending_reduce:
                b.reduce_grads(self.last_microbatch, self.async_grad_reduce, force=True)
        if self.last_microbatch or not self.async_grad_reduce:
            for b in self.buckets:
                if b.numel:
                    b.finish_reduce(self.async_grad_reduce)

    def finish_step(self) -> None:
        """End of an iteration: reduce the buckets whose reduction was deferred past the pipeline schedule."""
        for b in self.buckets:
            if b.numel and b.deferred and b.pending_reduce:
                for hook in b.pre_reduce_hooks:
                    hook()
                b.deferred = False
                b.reduce_grads(True, self.async_grad_reduce, force=True)
                b.finish_reduce(True)
                b.deferred = True

    def grad_norm(self) -> torch.Tensor:
        dev = next((b.device for b in self.buckets if b.numel), torch.device("cpu"))
        total = torch.zeros(1, dtype=torch.float32, device=dev)
        for b in self.buckets:
            tp = b.tp_group.size if b.tp_group is not None else 1
            b.grad_sumsq(total, tp)
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(total, group=self.world_group)
        return total.sqrt()

    def step(self, lr: float, beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8, weight_decay: float = 0.0,
             max_grad_norm: float = 0.0, loss_scale: float = 1.0):
        """One AdamW step over every bucket. ``loss_scale`` is what the losses were multiplied by before backward: it
        is divided out through the same device-side coefficient as the gradient clip, and a step whose (unscaled)
        global gradient norm is not finite is skipped on every rank (``last_step_skipped``)."""
        get_tracer().begin("optimizer_step", "optimizer")
        clip_coef, norm = None, None
        scaled = loss_scale != 1.0
        self.last_step_skipped = False
        if scaled or (max_grad_norm and max_grad_norm > 0):
            norm = self.grad_norm()
            if scaled:
                norm = norm / loss_scale
                if not bool(torch.isfinite(norm).all()):      # same value on every rank: the norm is a job-wide sum
                    self.last_step_skipped = True
                    self.last_norm = norm
                    get_tracer().end("optimizer_step")
                    return norm
            if max_grad_norm and max_grad_norm > 0:
                clip_coef = torch.clamp(max_grad_norm / (norm + 1e-6), max=1.0)
            else:
                clip_coef = torch.ones_like(norm)
            if scaled:
                clip_coef = clip_coef / loss_scale
        self.step_count += 1
        for b in self.buckets:
            b.step(lr, beta1, beta2, eps, weight_decay, self.step_count, clip_coef)
        get_tracer().end("optimizer_step")
        self.last_norm = norm
        self.check_guard_zones()
        return norm

    def check_guard_zones(self) -> None:
        """Debug mode (GV_SYMM_CANARY=1): nothing may have stored outside the payload regions of the buckets' peer-mapped
        allocations during the step (synchronises the device)."""
        from .symm import canaries_enabled

        if not canaries_enabled():
            return
        torch.cuda.synchronize()
        for b in self.buckets:
            f = getattr(b, "fused", None)
            if f is not None and f.ws.canary is not None:
                f.ws.canary.check("bucket " + b.name)

    def zero_grad(self) -> None:
        for b in self.buckets:
            b.zero_grad()

    def state_dict(self) -> dict:
        return {"step": self.step_count, "buckets": {b.name: b.state_dict() for b in self.buckets if b.numel}}

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = sd["step"]
        for b in self.buckets:
            if b.numel and b.name in sd["buckets"]:
                b.load_state_dict(sd["buckets"][b.name])
