"""Context parallelism: zigzag ring attention (rank c of cp owns sequence chunks c and 2cp-1-c of 2cp).

Reference: galvatron/core/runtime/tensor_parallel/transformer.py:2252-2327 (``RingComm``), :2335-2420 (forward with
the causal / first-half-KV / second-half-Q cases and the log-sum-exp merge :2208-2249), :2423-2551 (backward that
circulates (k, dk), (v, dv)).

Here step t of the ring works on the K/V block of rank (r - t): on an NVSwitch box every peer is one hop away, so
the block is fetched from its owner directly instead of being handed around. While the attention kernel works on
the current block the next one is already on its way into the second of two staging buffers, so at most two K/V
blocks besides the rank's own are resident (O(s / cp) memory). Partial outputs are merged by log-sum-exp in fp32
(``gv_lse_merge``). In the backward pass the block is fetched again, and the dK/dV a rank computes for the block of
rank (r - t) goes back to that owner, which adds the contributions of all steps in fp32. Only the rows a step really
uses travel: a step that attends to the first half of a block fetches, and returns gradients for, that half only.

Transports: ``nccl`` (and gloo on CPU ranks) uses batched isend/irecv; ``fused`` publishes the block once in the
group's symmetric memory and lets each consumer pull it with this package's peer-copy kernel on a side stream.
"""
from __future__ import annotations

from typing import List, Tuple

import torch
import torch.distributed as dist

from ..ops import autograd as A
from ..ops import functional as Fn


def ring_cases(cp: int, rank: int, causal: bool) -> List[Tuple[int, str]]:
    """Per step t: (owner of the K/V block, case). Cases: "diag" = own block, causal over the local (early, late)
    pair; "kv_first" = every local query row against the first half of the block (the owner's early chunk, which
    precedes both local chunks); "q_second" = the local late chunk against the whole block (an owner further down the
    sequence than the local early chunk); "full" = no mask (non-causal models)."""
    out = []
    for t in range(cp):
        src = (rank - t) % cp
        if not causal:
            out.append((src, "full"))
        elif t == 0:
            out.append((src, "diag"))
        elif t <= rank:
            out.append((src, "kv_first"))
        else:
            out.append((src, "q_second"))
    return out


# ------------------------------------------------------------------------------------------ transports
class _P2PRing:
    """K/V blocks and gradient blocks as batched point-to-point messages (NCCL on GPUs, gloo on CPU ranks)."""

    def __init__(self, cg, rank: int):
        self.cg, self.rank, self.cp = cg, rank, cg.size

    def begin(self, kv: torch.Tensor) -> None:
        self.kv = kv

    def fetch(self, t: int, rows_me: int, rows_peer: int, like: torch.Tensor):
        """Step t: this rank needs ``rows_me`` leading rows of the block of rank (r - t); rank (r + t) needs
        ``rows_peer`` leading rows of this rank's block. Returns a handle whose ``wait`` yields the received rows."""
        src, dst = self.cg.ranks[(self.rank - t) % self.cp], self.cg.ranks[(self.rank + t) % self.cp]
        buf = torch.empty((rows_me,) + tuple(like.shape[1:]), dtype=like.dtype, device=like.device)
        ops = [dist.P2POp(dist.isend, self.kv[:rows_peer].contiguous(), dst, group=self.cg.group),
               dist.P2POp(dist.irecv, buf, src, group=self.cg.group)]
        reqs = dist.batch_isend_irecv(ops)
        return _Handle(buf, reqs, keep=ops)

    def give_back(self, t: int, contrib: torch.Tensor, rows_in: int, like: torch.Tensor):
        """Step t of the backward pass: ``contrib`` (gradient rows of the block of rank (r - t)) goes to its owner;
        the contribution of rank (r + t) to this rank's block (``rows_in`` leading rows) comes back."""
        dst, src = self.cg.ranks[(self.rank - t) % self.cp], self.cg.ranks[(self.rank + t) % self.cp]
        buf = torch.empty((rows_in,) + tuple(like.shape[1:]), dtype=contrib.dtype, device=like.device)
        ops = [dist.P2POp(dist.isend, contrib.contiguous(), dst, group=self.cg.group),
               dist.P2POp(dist.irecv, buf, src, group=self.cg.group)]
        reqs = dist.batch_isend_irecv(ops)
        return _Handle(buf, reqs, keep=ops)

    def end(self) -> None:
        pass


class _Handle:
    def __init__(self, buf, reqs=(), event=None, keep=None):
        self.buf, self.reqs, self.event, self.keep = buf, list(reqs), event, keep

    def wait(self) -> torch.Tensor:
        for r in self.reqs:
            r.wait()
        if self.event is not None:
            torch.cuda.current_stream().wait_event(self.event)
        self.reqs, self.event, self.keep = [], None, None
        return self.buf


_PULL_STREAMS = {}


class _PeerPullRing:
    """K/V blocks published once in symmetric memory and pulled by their consumers on a side stream; gradient
    blocks published per step and pulled by the block's owner (csrc/nvlink_bench.cu ``p2p_pull_kernel``)."""

    def __init__(self, cg, rank: int, nbytes: int, tag: str):
        from . import fused

        self.cg, self.rank, self.cp = cg, rank, cg.size
        # a few dozen CTAs keep NVLink busy and leave the SMs to the attention kernel the transfer runs beside
        self.kv_box = fused.Mailbox(cg, nbytes, tag + "_kv", pull_blocks=48)
        self.g_box = fused.Mailbox(cg, nbytes, tag + "_dkv", pull_blocks=48)
        dev = torch.cuda.current_device()
        if dev not in _PULL_STREAMS:
            _PULL_STREAMS[dev] = torch.cuda.Stream()
        self.side = _PULL_STREAMS[dev]

    def begin(self, kv: torch.Tensor) -> None:
        self.kv = kv
        self.kv_box.publish(kv)

    def fetch(self, t: int, rows_me: int, rows_peer: int, like: torch.Tensor):
        buf = torch.empty((rows_me,) + tuple(like.shape[1:]), dtype=like.dtype, device=like.device)
        self.side.wait_stream(torch.cuda.current_stream())     # the staging memory may still be read by earlier kernels
        with torch.cuda.stream(self.side):
            self.kv_box.pull((self.rank - t) % self.cp, buf)
            ev = self.side.record_event()
        buf.record_stream(self.side)
        return _Handle(buf, event=ev)

    def give_back(self, t: int, contrib: torch.Tensor, rows_in: int, like: torch.Tensor):
        # the owner of the block, rank (r - t), is the one reader of this publication
        self.g_box.publish(contrib.contiguous(), readers=[(self.rank - t) % self.cp])
        buf = torch.empty((rows_in,) + tuple(like.shape[1:]), dtype=contrib.dtype, device=like.device)
        self.g_box.pull((self.rank + t) % self.cp, buf)
        return _Handle(buf)

    def end(self) -> None:
        # every rank pulls from every other rank in each call, so the next call's publication (two epochs after the
        # buffer's last use) needs no barrier: see fused.Mailbox
        torch.cuda.current_stream().wait_stream(self.side)


def _make_ring(cg, rank: int, kv: torch.Tensor, impl: str, tag: str):
    if impl == "fused" and kv.is_cuda and kv.dtype == torch.bfloat16 and (kv.numel() * 2) % 32 == 0:
        from . import symm
        if symm.available(cg):
            return _PeerPullRing(cg, rank, kv.numel() * 2, tag)
    return _P2PRing(cg, rank)


# ------------------------------------------------------------------------------------------ the ring
def _views(q, kv_rows, hk: int, dh: int):
    """q [s, b, hq, dh] -> [b, s, hq, dh]; packed kv rows [rows, b, 2 hk dh] -> k, v [b, rows, hk, dh] (views)."""
    rows, b = kv_rows.shape[0], kv_rows.shape[1]
    k = kv_rows[..., : hk * dh].view(rows, b, hk, dh).transpose(0, 1)
    v = kv_rows[..., hk * dh:].view(rows, b, hk, dh).transpose(0, 1)
    return q.transpose(0, 1), k, v


def _rows_needed(case: str, s_loc: int) -> int:
    return s_loc // 2 if case == "kv_first" else s_loc


class ZigzagRingAttention(torch.autograd.Function):
    """q [s_loc, b, hq, dh], kv [s_loc, b, 2 hk dh] (k | v packed, RoPE already applied) -> o [s_loc, b, hq, dh]."""

    @staticmethod
    def forward(ctx, q, kv, cg, rank, impl, causal, scale, hk):
        cp = cg.size
        s_loc, b, hq, dh = q.shape
        half = s_loc // 2
        cases = ring_cases(cp, rank, causal)
        ring = _make_ring(cg, rank, kv, impl, "cp%d_%d" % (s_loc * b, 2 * hk * dh))
        kv = kv.contiguous()
        ring.begin(kv)
        acc = torch.zeros(b, s_loc, hq, dh, dtype=torch.float32, device=q.device)
        lse = torch.full((b, hq, s_loc), float("-inf"), dtype=torch.float32, device=q.device)
        nxt = None
        for t, (src, case) in enumerate(cases):
            blk = kv if t == 0 else nxt.wait()
            if t + 1 < cp:
                # the next block travels while this one is computed on; how many of this rank's rows its consumer
                # (rank r + t + 1) needs follows from that rank's case at the same step
                peer_case = ring_cases(cp, (rank + t + 1) % cp, causal)[t + 1][1]
                nxt = ring.fetch(t + 1, _rows_needed(cases[t + 1][1], s_loc), _rows_needed(peer_case, s_loc), kv)
            q_rows = q[half:] if case == "q_second" else q
            qb, kb, vb = _views(q_rows, blk, hk, dh)
            o_blk, lse_blk = Fn.attention_fwd(qb, kb, vb, case == "diag", scale)
            Fn.lse_merge_(acc, lse, o_blk, lse_blk, half if case == "q_second" else 0)
        ring.end()
        out = acc.to(q.dtype)                                   # [b, s_loc, hq, dh]
        ctx.cg, ctx.rank, ctx.impl, ctx.causal, ctx.scale, ctx.hk = cg, rank, impl, causal, scale, hk
        ctx.save_for_backward(q, kv, out, lse)
        return out.transpose(0, 1)

    @staticmethod
    def backward(ctx, dout):
        q, kv, out, lse = ctx.saved_tensors
        cg, rank, impl, causal, scale, hk = ctx.cg, ctx.rank, ctx.impl, ctx.causal, ctx.scale, ctx.hk
        cp = cg.size
        s_loc, b, hq, dh = q.shape
        half = s_loc // 2
        cases = ring_cases(cp, rank, causal)
        ring = _make_ring(cg, rank, kv, impl, "cp%d_%d" % (s_loc * b, 2 * hk * dh))
        ring.begin(kv)
        do = dout.transpose(0, 1)                               # [b, s_loc, hq, dh]
        dq = torch.zeros(b, s_loc, hq, dh, dtype=torch.float32, device=q.device)
        dkv = torch.zeros(kv.shape, dtype=torch.float32, device=q.device)
        lse_late = lse[:, :, half:].contiguous() if causal and cp > 1 else None
        nxt = None
        for t, (src, case) in enumerate(cases):
            blk = kv if t == 0 else nxt.wait()
            if t + 1 < cp:
                peer_case = ring_cases(cp, (rank + t + 1) % cp, causal)[t + 1][1]
                nxt = ring.fetch(t + 1, _rows_needed(cases[t + 1][1], s_loc), _rows_needed(peer_case, s_loc), kv)
            late = case == "q_second"
            q_rows = q[half:] if late else q
            qb, kb, vb = _views(q_rows, blk, hk, dh)
            sl = slice(half, None) if late else slice(None)
            dq_p, dk_p, dv_p = Fn.attention_bwd(do[:, sl], qb, kb, vb, out[:, sl], lse_late if late else lse, case == "diag", scale)
            dq[:, sl] += dq_p.float()
            contrib = torch.cat([dk_p.transpose(0, 1).reshape(blk.shape[0], b, hk * dh),
                                 dv_p.transpose(0, 1).reshape(blk.shape[0], b, hk * dh)], dim=-1)
            if t == 0:
                dkv += contrib.float()
            else:
                # the contribution that comes back is the one rank (r + t) computed at ITS step t for this rank's block
                rows_in = _rows_needed(ring_cases(cp, (rank + t) % cp, causal)[t][1], s_loc)
                got = ring.give_back(t, contrib, rows_in, kv).wait()
                dkv[:rows_in] += got.float()
        ring.end()
        return dq.to(q.dtype).transpose(0, 1), dkv.to(kv.dtype), None, None, None, None, None, None


def ring_attention_packed(qkv: torch.Tensor, attn_module, ctx, causal: bool, rope: bool) -> torch.Tensor:
    st, cfg = attn_module.st, attn_module.cfg
    cp, r = st.cp, st.cp_rank
    hq, hk, dh = attn_module.hq_w, attn_module.hk_w, cfg.head_dim
    b = ctx.batch
    s_loc = qkv.shape[0] // b
    chunk = s_loc // 2
    x = qkv.view(s_loc, b, (hq + 2 * hk) * dh)
    q = x[..., : hq * dh].reshape(s_loc, b, hq, dh)
    k = x[..., hq * dh:(hq + hk) * dh].reshape(s_loc, b, hk, dh)
    v = x[..., (hq + hk) * dh:].reshape(s_loc, b, hk, dh)
    if rope:
        pos_s = torch.cat([torch.arange(r * chunk, (r + 1) * chunk, device=qkv.device),
                           torch.arange((2 * cp - 1 - r) * chunk, (2 * cp - r) * chunk, device=qkv.device)])
        positions = pos_s.view(s_loc, 1).expand(s_loc, b).reshape(-1)
        q = A.rope(q.reshape(s_loc * b, hq, dh), attn_module.inv_freq, 1, 0, 0, positions).view(s_loc, b, hq, dh)
        k = A.rope(k.reshape(s_loc * b, hk, dh), attn_module.inv_freq, 1, 0, 0, positions).view(s_loc, b, hk, dh)
    kv = torch.cat([k.reshape(s_loc, b, hk * dh), v.reshape(s_loc, b, hk * dh)], dim=-1)
    scale = 1.0 / (dh ** 0.5)
    o = ZigzagRingAttention.apply(q, kv, st.cp_group, r, st.impl, causal, scale, hk)      # [s_loc, b, hq, dh]
    return o.reshape(s_loc * b, hq * dh)


def kv_residency_bytes(seq: int, batch: int, hk: int, dh: int, cp: int, elem: int = 2) -> dict:
    """K/V bytes resident per rank and layer during the attention call: the ring keeps the own block and two staging
    blocks; gathering the whole sequence up front (what this module did before) keeps all cp blocks."""
    block = seq // cp * batch * 2 * hk * dh * elem
    return {"ring": 3 * block, "gather_all": (cp + 1) * block}
