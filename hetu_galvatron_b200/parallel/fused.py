"""Host side of the fused compute + collective paths (``--comm_impl fused``).

Each function is the drop-in counterpart of a library-collective sequence in ``ops/autograd.py`` /
``parallel/ulysses.py`` / ``parallel/reshard.py`` / ``parallel/zero.py`` and is validated against it
(tests/test_fused_gpu.py):

===========================  =============================================  ====================================
function                     replaces                                       kernels
===========================  =============================================  ====================================
allgather_gemm               all_gather(x) ; x W^T                          gv_fused_gemm (a_mode 1)
gemm_reduce                  x W^T ; reduce_scatter / all_reduce            gv_fused_gemm (c_mode 1) + gv_reduce_slots
qkv_to_heads / heads_to_out  Ulysses projections + all-to-alls              gv_fused_gemm (c_mode 2 / a_mode 2)
reshard                      all_gather over the stage ; slice              gv_reshard_gather
allgather_pull               all_gather_into_tensor (ZeRO-3 parameters)     gv_allgather_pull
rs_adamw                     reduce_scatter ; AdamW ; all_gather            gv_rs_adamw
===========================  =============================================  ====================================

Workspaces are double buffered by epoch parity: a rank reuses the buffer of epoch e-2 only after it has seen every
peer's epoch e-1 announcement, which each peer makes after it finished reading epoch e-2 (stream order).
"""
from __future__ import annotations

import ctypes
import weakref
from typing import Dict, Optional

import torch

from ..ops import _lib
from .mesh import CommGroup
from .symm import FusedGemmArgs, SymmWorkspace, canaries_enabled, check_canaries, workspace

SLOT_AG, SLOT_RS, SLOT_AR, SLOT_U1, SLOT_U2, SLOT_RESHARD, SLOT_PARAM, SLOT_GRAD = 0, 1, 2, 3, 4, 5, 6, 7

_GROUPS: Dict[int, CommGroup] = {}
# Ulysses column maps, one per send-column index tensor: keyed by the tensor's id, guarded by a weak reference to the
# tensor itself, so the entry dies with the tensor and a new tensor at a recycled address never sees a stale map
_COL_MAPS: Dict[int, tuple] = {}


def _col_map_get(idx: torch.Tensor):
    entry = _COL_MAPS.get(id(idx))
    return entry[1] if entry is not None and entry[0]() is idx else None


def _col_map_put(idx: torch.Tensor, col_map: torch.Tensor) -> None:
    key = id(idx)
    _COL_MAPS[key] = (weakref.ref(idx, lambda _ref, key=key: _COL_MAPS.pop(key, None)), col_map)


def register_group(cg: CommGroup) -> None:
    if cg.group is not None:
        _GROUPS[id(cg.group)] = cg


def comm_group(pg) -> CommGroup:
    cg = _GROUPS.get(id(pg))
    if cg is None:
        raise RuntimeError("process group was not created through Mesh.group(); the fused paths need its rank list")
    return cg


def _guarded(fn):
    """Debug mode (GV_SYMM_CANARY=1): after the collective, verify the guard zones of every cached workspace."""
    import functools

    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        out = fn(*args, **kwargs)
        if canaries_enabled():
            check_canaries(fn.__name__)
        return out

    return wrapper


def _sp(stream=None):
    return ctypes.c_void_p(_lib.stream_ptr())


def _lib_fused():
    lib = _lib.lib()
    return lib


def _bf16_2d(t: torch.Tensor) -> torch.Tensor:
    if t.dtype != torch.bfloat16 or not t.is_cuda:
        raise _lib.KernelError("fused communication kernels need bf16 CUDA tensors")
    t = t.reshape(-1, t.shape[-1])
    return t if t.is_contiguous() else t.contiguous()


def _act_workspace(cg: CommGroup, rows_loc: int, width: int) -> SymmWorkspace:
    """Workspace for [rows_loc, width] activations of a tp group: 2 gather buffers + 2 x world scatter slots."""
    per = rows_loc * width * 2
    need = per * 2 + per * cg.size * 2 + per * 2 + 4096
    return workspace(cg, need, tag="act_%d_%d" % (rows_loc, width))


# ------------------------------------------------------------------------------------------ F1
@_guarded
def allgather_gemm(x2: torch.Tensor, W: torch.Tensor, pg, bias: Optional[torch.Tensor] = None,
                   return_gathered: bool = False, b_mn: bool = False):
    """y[world * rows, N] = all_gather_rows(x2) @ W^T (+ bias). Copy warps inside the GEMM kernel pull the peers' row
    blocks once into a local buffer while the tensor cores work on the own rows; with ``return_gathered`` that buffer
    (the gathered activation, own rows filled in) is returned too, for the weight-gradient GEMM of the backward pass.
    ``b_mn``: W is used as stored [K, N] (input-gradient GEMM of a row-parallel layer)."""
    cg = comm_group(pg)
    x2 = _bf16_2d(x2)
    rows, K = x2.shape
    N = W.shape[1] if b_mn else W.shape[0]
    if rows % 128 != 0 or K % 8 != 0:
        raise _lib.KernelError("allgather_gemm needs a per-rank row count divisible by 128")
    ws = _act_workspace(cg, rows, K)
    e = ws.next_epoch(SLOT_AG)
    off = ws.region("ag%d" % (e & 1), rows * K * 2)
    ws.view(off, (rows, K)).copy_(x2)
    ws.signal(SLOT_AG, e)
    M = rows * cg.size
    out = torch.empty(M, N, dtype=x2.dtype, device=x2.device)
    gathered = torch.empty(M, K, dtype=x2.dtype, device=x2.device)
    counters = torch.zeros(M // 128, dtype=torch.int32, device=x2.device)
    a = FusedGemmArgs(A=None, B=W.data_ptr(), C=out.data_ptr(), bias=_lib.p(bias), M=M, N=N, K=K, lda=K, ldb=W.stride(0),
                      ldc=N, a_mode=1, c_mode=0, a_off=off, c_off=0, slot_in=SLOT_AG, slot_out=-1, epoch=e,
                      gather_buf=gathered.data_ptr(), gather_ctr=counters.data_ptr())
    _lib.check(_lib.lib().gv_fused_gemm_ex(ctypes.byref(ws.peers), ctypes.byref(a), int(b_mn), None, 0, _sp()), "gv_fused_gemm(ag)")
    if return_gathered:
        r = ws.rank
        gathered[r * rows:(r + 1) * rows].copy_(x2)
        return out, gathered
    return out


# ------------------------------------------------------------------------------------------ F2 / F3
@_guarded
def gemm_reduce(x2: torch.Tensor, W: torch.Tensor, pg, scatter: bool = True, residual: Optional[torch.Tensor] = None,
                bias: Optional[torch.Tensor] = None, b_mn: bool = False) -> torch.Tensor:
    """Row-parallel GEMM fused with its reduction: every output tile is stored straight into the owner rank's slot;
    the owner sums the slots (+ residual + bias). ``scatter=False`` additionally gathers the reduced rows (all-reduce).
    ``b_mn``: W is used as stored [K_red, N_out] (input-gradient GEMM of a column-parallel layer)."""
    cg = comm_group(pg)
    x2 = _bf16_2d(x2)
    M, K = x2.shape
    N = W.shape[1] if b_mn else W.shape[0]
    t = cg.size
    rows = M // t
    if M % t or N % 8 or K % 8:
        raise _lib.KernelError("gemm_reduce: shape not supported (M %% world, N %% 8, K %% 8)")
    ws = _act_workspace(cg, rows, N)
    e = ws.next_epoch(SLOT_RS)
    off = ws.region("rs%d" % (e & 1), t * rows * N * 2)
    a = FusedGemmArgs(A=x2.data_ptr(), B=W.data_ptr(), C=None, bias=None, M=M, N=N, K=K, lda=x2.stride(0), ldb=W.stride(0),
                      ldc=N, a_mode=0, c_mode=1, a_off=0, c_off=off, slot_in=-1, slot_out=SLOT_RS, epoch=e)
    _lib.check(_lib.lib().gv_fused_gemm_ex(ctypes.byref(ws.peers), ctypes.byref(a), int(b_mn), None, 0, _sp()), "gv_fused_gemm(rs)")
    if scatter:
        out = torch.empty(rows, N, dtype=x2.dtype, device=x2.device)
        res = None if residual is None else _bf16_2d(residual)
        _lib.check(_lib.lib().gv_reduce_slots(ctypes.byref(ws.peers), ctypes.c_longlong(off), ctypes.c_void_p(out.data_ptr()),
                                              ctypes.c_void_p(_lib.p(res)), ctypes.c_void_p(_lib.p(bias)),
                                              ctypes.c_longlong(rows), N, SLOT_RS, ctypes.c_uint(e), _sp()), "gv_reduce_slots")
        return out
    # all-reduce: reduce my row block into a gather buffer, announce it, pull everyone's block
    e2 = ws.next_epoch(SLOT_AR)
    goff = ws.region("ar%d" % (e2 & 1), rows * N * 2)
    mine = ws.view(goff, (rows, N))
    _lib.check(_lib.lib().gv_reduce_slots(ctypes.byref(ws.peers), ctypes.c_longlong(off), ctypes.c_void_p(mine.data_ptr()),
                                          None, None, ctypes.c_longlong(rows), N, SLOT_RS, ctypes.c_uint(e), _sp()), "gv_reduce_slots")
    ws.signal(SLOT_AR, e2)
    out = torch.empty(M, N, dtype=x2.dtype, device=x2.device)
    _lib.check(_lib.lib().gv_allgather_pull(ctypes.byref(ws.peers), ctypes.c_longlong(goff), ctypes.c_void_p(out.data_ptr()),
                                            ctypes.c_longlong(rows * N), SLOT_AR, ctypes.c_uint(e2), _sp()), "gv_allgather_pull")
    if bias is not None:
        out += bias
    if residual is not None:
        out += residual.reshape(out.shape)
    return out


# ------------------------------------------------------------------------------------------ pull all-gather
@_guarded
def allgather_pull(shard: torch.Tensor, cg: CommGroup, tag: str, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """All-gather of equal 2-byte-element shards by pulling from peer memory (ZeRO-3 parameter gather, backward
    activation gathers). The shard is staged in the symmetric workspace of (group, tag)."""
    n = shard.numel()
    ws = workspace(cg, 2 * n * 2 + 4096, tag="agp_%s_%d" % (tag, n))
    e = ws.next_epoch(SLOT_PARAM)
    off = ws.region("p%d" % (e & 1), n * 2)
    ws.view(off, (n,), shard.dtype).copy_(shard.reshape(-1))
    ws.signal(SLOT_PARAM, e)
    if out is None:
        out = torch.empty(cg.size * n, dtype=shard.dtype, device=shard.device)
    _lib.check(_lib.lib().gv_allgather_pull(ctypes.byref(ws.peers), ctypes.c_longlong(off), ctypes.c_void_p(out.data_ptr()),
                                            ctypes.c_longlong(n), SLOT_PARAM, ctypes.c_uint(e), _sp()), "gv_allgather_pull")
    return out


# ------------------------------------------------------------------------------------------ plain NVLink collectives
SLOT_NVL_A, SLOT_NVL_B = 8, 9


def p2p_pull(buf: torch.Tensor, src: int, cg: CommGroup, tag: str = "p2p") -> torch.Tensor:
    """Every rank publishes ``buf`` and pulls peer ``src``'s copy (send/recv over NVLink as a one-sided read)."""
    n = buf.numel() * buf.element_size()
    ws = workspace(cg, 2 * n + 4096, tag="nvl_%s_%d" % (tag, n))
    e = ws.next_epoch(SLOT_NVL_A)
    off = ws.region("b%d" % (e & 1), n)
    ws.buffer[off:off + n].copy_(buf.reshape(-1).view(torch.uint8))
    ws.signal(SLOT_NVL_A, e)
    out = torch.empty_like(buf)
    _lib.check(_lib.lib().gv_p2p_pull(ctypes.byref(ws.peers), src, ctypes.c_longlong(off), ctypes.c_void_p(out.data_ptr()),
                                      ctypes.c_longlong(n), SLOT_NVL_A, ctypes.c_uint(e), _sp()), "gv_p2p_pull")
    # the pull only waits for its source; the rank that reads THIS rank's buffer may be another one, so the
    # double-buffer rule (reuse of epoch e-2 only after every peer announced e-1) needs every reader's word
    ws.barrier(SLOT_NVL_B)
    return out


@_guarded
def alltoall_pull(buf: torch.Tensor, cg: CommGroup, tag: str = "a2a") -> torch.Tensor:
    """``all_to_all_single`` with equal splits: block s of the result is peer s's block ``rank``."""
    n = buf.numel() * buf.element_size()
    ws = workspace(cg, 2 * n + 4096, tag="nvl_%s_%d" % (tag, n))
    e = ws.next_epoch(SLOT_NVL_A)
    off = ws.region("b%d" % (e & 1), n)
    ws.buffer[off:off + n].copy_(buf.reshape(-1).view(torch.uint8))
    ws.signal(SLOT_NVL_A, e)
    out = torch.empty_like(buf)
    _lib.check(_lib.lib().gv_alltoall_pull(ctypes.byref(ws.peers), ctypes.c_longlong(off), ctypes.c_void_p(out.data_ptr()),
                                           ctypes.c_longlong(n // cg.size), SLOT_NVL_A, ctypes.c_uint(e), _sp()), "gv_alltoall_pull")
    return out


def allreduce_symm(buf: torch.Tensor, cg: CommGroup, tag: str = "ar", multimem: bool = False) -> torch.Tensor:
    """Two-shot all-reduce of a bf16 tensor staged in symmetric memory: every rank reduces one shard over all peers
    and writes it back to all of them; ``multimem`` does both inside NVSwitch (needs a multicast mapping)."""
    if buf.dtype != torch.bfloat16 or buf.numel() % (8 * cg.size):
        raise _lib.KernelError("allreduce_symm needs bf16 with numel divisible by 8 * world")
    n = buf.numel() * 2
    ws = workspace(cg, 2 * n + 4096, tag="nvl_%s_%d" % (tag, n))
    if multimem and not ws.multicast_ptr:
        raise _lib.KernelError("no multicast mapping available for this group")
    e = ws.next_epoch(SLOT_NVL_A)
    off = ws.region("b%d" % (e & 1), n)
    stage = ws.view(off, (buf.numel(),))
    stage.copy_(buf.reshape(-1))
    ws.signal(SLOT_NVL_A, e)
    mc = ctypes.c_void_p(ws.multicast_ptr) if multimem else None
    _lib.check(_lib.lib().gv_allreduce_shard(ctypes.byref(ws.peers), mc, ctypes.c_longlong(off), ctypes.c_longlong(buf.numel()),
                                             SLOT_NVL_A, ctypes.c_uint(e), _sp()), "gv_allreduce_shard")
    ws.barrier(SLOT_NVL_B)
    return stage.view(buf.shape).clone()


class Mailbox:
    """A double-buffered region of a group's symmetric memory that every rank can publish a tensor into and any peer
    can then pull from (send / recv as one-sided reads): the transport of the context-parallel ring, where step t needs
    the block of rank (r - t), every peer being one NVSwitch hop away.

    ``publish`` stages the tensor and announces a new epoch; ``pull(src, ...)`` copies (part of) peer ``src``'s current
    publication into a local tensor once ``src`` has announced it. Publication e + 1 overwrites the buffer of e - 1;
    that is safe once every reader of e - 1 has announced its own epoch e (a rank announces e only after, in stream
    order, it finished reading e - 1). ``publish(readers=...)`` names the ranks that will read this publication; the
    next use of the same buffer waits for exactly those ranks (None: the caller guarantees it otherwise, e.g. because
    it pulls from every peer in every epoch)."""

    def __init__(self, cg: CommGroup, max_bytes: int, tag: str, pull_blocks: int = 0):
        self.max_bytes = (max_bytes + 255) // 256 * 256
        self.ws = workspace(cg, 2 * self.max_bytes + 4096, tag="mbox_%s_%d" % (tag, self.max_bytes))
        self.cg = cg
        self.off = 0
        self.epoch = 0
        self.pull_blocks = pull_blocks
        if not hasattr(self.ws, "_mbox_readers"):
            self.ws._mbox_readers = {}          # buffer parity -> (epoch, ranks that read that publication)

    def publish(self, t: torch.Tensor, readers=None) -> None:
        n = t.numel() * t.element_size()
        assert n <= self.max_bytes and n % 16 == 0
        ws = self.ws
        self.epoch = ws.next_epoch(SLOT_NVL_A)
        parity = self.epoch & 1
        prev = ws._mbox_readers.get(parity)
        if prev is not None and prev[1]:
            for r in prev[1]:                    # the ranks that read epoch e - 2 have announced e - 1 since
                if r != ws.rank:
                    ws.wait(SLOT_NVL_A, r, prev[0] + 1)
        ws._mbox_readers[parity] = (self.epoch, list(readers) if readers is not None else None)
        self.off = ws.region("b%d" % parity, self.max_bytes)
        ws.buffer[self.off:self.off + n].copy_(t.reshape(-1).view(torch.uint8))
        ws.signal(SLOT_NVL_A, self.epoch)

    def pull(self, src: int, out: torch.Tensor, nbytes: Optional[int] = None, src_byte_offset: int = 0) -> torch.Tensor:
        n = out.numel() * out.element_size() if nbytes is None else nbytes
        _lib.check(_lib.lib().gv_p2p_pull_ex(ctypes.byref(self.ws.peers), src, ctypes.c_longlong(self.off + src_byte_offset),
                                             ctypes.c_void_p(out.data_ptr()), ctypes.c_longlong(n), SLOT_NVL_A,
                                             ctypes.c_uint(self.epoch), self.pull_blocks, _sp()), "gv_p2p_pull")
        return out

    def release(self) -> None:
        self.ws.barrier(SLOT_NVL_B)


# ------------------------------------------------------------------------------------------ Z2
def rs_adamw(grad: torch.Tensor, master: torch.Tensor, exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor, cg: CommGroup, *,
             step: int, lr: float, beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8, weight_decay: float = 0.0,
             grad_scale: float = 1.0, clip_coef: Optional[torch.Tensor] = None, sumsq_out: Optional[torch.Tensor] = None,
             tag: str = "zero") -> torch.Tensor:
    """Gradient reduce-scatter + AdamW + parameter all-gather in one kernel: every rank publishes its full gradient
    bucket ``grad`` [n] (bf16 or fp32), sums its own shard over all peers, updates ``master`` / moments (fp32 shards of
    n / world elements) and writes the new bf16 parameters of its shard into EVERY rank's parameter buffer. Returns
    the full updated bf16 parameter vector [n] (a view of the workspace, valid until the next call with this tag)."""
    n, w = grad.numel(), cg.size
    if n % (4 * w) or master.numel() * w != n:
        raise _lib.KernelError("rs_adamw needs numel divisible by 4 * world and fp32 shards of numel / world")
    gbytes = n * grad.element_size()
    ws = workspace(cg, 2 * gbytes + n * 2 + 8192, tag="z2_%s_%d_%d" % (tag, n, grad.element_size()))
    e = ws.next_epoch(SLOT_GRAD)
    goff = ws.region("g%d" % (e & 1), gbytes)
    poff = ws.region("params", n * 2)
    ws.buffer[goff:goff + gbytes].copy_(grad.reshape(-1).view(torch.uint8))
    ws.signal(SLOT_GRAD, e)
    shard = n // w
    bc1, bc2 = 1.0 - beta1 ** step, 1.0 - beta2 ** step
    _lib.check(_lib.lib().gv_rs_adamw(
        ctypes.byref(ws.peers), ctypes.c_longlong(goff), int(grad.dtype == torch.bfloat16), ctypes.c_longlong(ws.rank * shard),
        ctypes.c_longlong(shard), ctypes.c_void_p(master.data_ptr()), ctypes.c_void_p(exp_avg.data_ptr()),
        ctypes.c_void_p(exp_avg_sq.data_ptr()), ctypes.c_longlong(poff), 1, ctypes.c_float(lr), ctypes.c_float(beta1),
        ctypes.c_float(beta2), ctypes.c_float(eps), ctypes.c_float(weight_decay), ctypes.c_float(bc1), ctypes.c_float(bc2),
        ctypes.c_float(grad_scale), ctypes.c_void_p(_lib.p(clip_coef)), ctypes.c_void_p(_lib.p(sumsq_out)), SLOT_GRAD,
        ctypes.c_uint(e), _sp()), "gv_rs_adamw")
    ws.barrier(SLOT_NVL_B)        # every rank's shard has landed in every parameter buffer
    return ws.view(poff, (n,))


# ------------------------------------------------------------------------------------------ U1 / U2
@_guarded
def qkv_to_heads(x2: torch.Tensor, W: torch.Tensor, bias, idx: torch.Tensor, cg: CommGroup) -> torch.Tensor:
    """Ulysses: QKV projection whose epilogue stores every head group's columns straight into the rank that owns
    that group, in sequence order: returns [world * rows_loc, c] = the full sequence for this rank's heads.
    ``idx`` [world, c] lists, per destination rank, the projection columns it receives."""
    x2 = _bf16_2d(x2)
    rows, K = x2.shape
    p, c = idx.shape
    N = W.shape[0]
    col_map = _col_map_get(idx)
    if col_map is None:
        # destination of every 32-column chunk of the projection output; columns sent to several ranks
        # (replicated KV heads) are not supported by the store-once epilogue
        dest = torch.full((N,), -1, dtype=torch.int64)
        flat = idx.cpu()
        for r in range(p):
            if (dest[flat[r]] >= 0).any():
                raise _lib.KernelError("fused Ulysses needs kv heads >= sp degree (no replicated KV heads)")
            dest[flat[r]] = r * (1 << 24) + torch.arange(c)
        chunks = dest.view(-1, 32)
        if (chunks[:, 0] < 0).any() or ((chunks - chunks[:, :1]) != torch.arange(32)).any():
            raise _lib.KernelError("fused Ulysses needs head dims that keep 32-column chunks contiguous")
        col_map = chunks[:, 0].to(torch.int32).to(x2.device)
        _col_map_put(idx, col_map)
    ws = workspace(cg, 2 * p * rows * c * 2 + 4096, tag="u1_%d_%d" % (rows, c))
    e = ws.next_epoch(SLOT_U1)
    off = ws.region("h%d" % (e & 1), p * rows * c * 2)
    a = FusedGemmArgs(A=x2.data_ptr(), B=W.data_ptr(), C=None, bias=_lib.p(bias), M=rows, N=N, K=K, lda=x2.stride(0),
                      ldb=W.stride(0), ldc=N, a_mode=0, c_mode=2, a_off=0, c_off=off, slot_in=-1, slot_out=SLOT_U1, epoch=e)
    _lib.check(_lib.lib().gv_fused_gemm_ex(ctypes.byref(ws.peers), ctypes.byref(a), 0, ctypes.c_void_p(col_map.data_ptr()), c, _sp()),
               "gv_fused_gemm(u1)")
    for src in range(p):
        ws.wait(SLOT_U1, src, e)
    # hand the attention kernel a private copy so the workspace can be reused two epochs later
    return ws.view(off, (p * rows, c)).clone()


@_guarded
def heads_to_out(o2: torch.Tensor, W: torch.Tensor, bias, residual, cg: CommGroup) -> torch.Tensor:
    """Ulysses: output projection whose A operand K-slices (head groups) are read from the ranks that computed them:
    y[rows_loc, h] = concat_r(o_r[my rows]) @ W^T (+ bias) (+ residual)."""
    o2 = _bf16_2d(o2)
    full_rows, k_per = o2.shape
    p = cg.size
    rows = full_rows // p
    N, K = W.shape
    ws = workspace(cg, 2 * full_rows * k_per * 2 + 4096, tag="u2_%d_%d" % (full_rows, k_per))
    e = ws.next_epoch(SLOT_U2)
    off = ws.region("o%d" % (e & 1), full_rows * k_per * 2)
    ws.view(off, (full_rows, k_per)).copy_(o2)
    ws.signal(SLOT_U2, e)
    out = torch.empty(rows, N, dtype=o2.dtype, device=o2.device)
    a = FusedGemmArgs(A=None, B=W.data_ptr(), C=out.data_ptr(), bias=_lib.p(bias), M=rows, N=N, K=K, lda=K, ldb=W.stride(0),
                      ldc=N, a_mode=2, c_mode=0, a_off=off, c_off=0, slot_in=SLOT_U2, slot_out=-1, epoch=e)
    _lib.check(_lib.lib().gv_fused_gemm_ex(ctypes.byref(ws.peers), ctypes.byref(a), 0, None, 0, _sp()), "gv_fused_gemm(u2)")
    if residual is not None:
        out += residual.reshape(out.shape)
    return out


# ------------------------------------------------------------------------------------------ R1
@_guarded
def reshard(x3: torch.Tensor, old, new, mesh, stage_batch: int, seq: int) -> torch.Tensor:
    """Inter-layer relayout in one gather kernel: this rank reads exactly the rows it needs from its peers."""
    from .reshard import source_map

    cg = mesh.group("stage")
    s_old, b_old, h = x3.shape
    n = s_old * b_old * h
    ws = workspace(cg, 2 * n * 2 + 4096, tag="rsh_%d_%d_%d" % (s_old, b_old, h))
    e = ws.next_epoch(SLOT_RESHARD)
    off = ws.region("x%d" % (e & 1), n * 2)
    ws.view(off, (s_old, b_old, h)).copy_(x3)
    ws.signal(SLOT_RESHARD, e)
    key = (old, new, mesh.local, stage_batch, seq, str(x3.device))
    maps = _RESHARD_MAPS.get(key)
    if maps is None:
        src_rank, src_row, src_col = source_map(old, new, mesh.local, mesh.stage_size, stage_batch, seq)
        maps = tuple(t.to(torch.int32).contiguous().to(x3.device) for t in (src_rank, src_row, src_col))
        _RESHARD_MAPS[key] = maps
    src_rank, src_row, src_col = maps
    s_new, b_new = src_rank.shape
    out = torch.empty(s_new, b_new, h, dtype=x3.dtype, device=x3.device)
    _lib.check(_lib.lib().gv_reshard_gather(ctypes.byref(ws.peers), ctypes.c_longlong(off), ctypes.c_void_p(out.data_ptr()),
                                            ctypes.c_void_p(src_rank.data_ptr()), ctypes.c_void_p(src_row.data_ptr()),
                                            ctypes.c_void_p(src_col.data_ptr()), s_new, b_new, b_old, h, SLOT_RESHARD,
                                            ctypes.c_uint(e), _sp()), "gv_reshard_gather")
    return out


_RESHARD_MAPS: Dict[tuple, tuple] = {}
