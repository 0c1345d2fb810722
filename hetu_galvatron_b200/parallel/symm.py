"""Symmetric peer-mapped workspaces for the fused compute + collective kernels.

A ``SymmWorkspace`` is a buffer of the same size on every rank of a group, mapped into every peer's address space
(allocation and handle exchange go through ``torch.distributed._symmetric_memory``, i.e. CUDA VMM + fabric/posix
handles underneath; the kernels that use it are this package's own, csrc/comm_kernels.cu and
csrc/fused_gemm_sm100.cu). Layout: [flag area | payload]; payload regions are handed out by a bump allocator so
offsets are identical on all ranks. Epoch counters advance in lock-step because every rank executes the same
sequence of collective calls.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..ops import _lib
from .mesh import CommGroup

FLAG_BYTES = 512
MAX_RANKS = 8
# Debug mode (GV_SYMM_CANARY=1): 256 bytes of a fixed pattern right behind the flag area and at the very end of every
# workspace. Nothing ever writes there, so a changed byte means some rank's kernel stored outside the payload regions
# it was given (an offset or extent bug in a peer-memory kernel); `check_canaries` reads them back and says where.
CANARY_BYTES = 256
CANARY_VALUE = 0xA5


def canaries_enabled() -> bool:
    return os.environ.get("GV_SYMM_CANARY", "0") == "1"


class CanaryGuard:
    """The two guard zones of one buffer (any uint8 tensor): ``arm`` writes the pattern, ``check`` raises with the first
    changed offset."""

    def __init__(self, buffer: torch.Tensor, head_off: int, tail_off: int, nbytes: int = CANARY_BYTES):
        assert buffer.dtype == torch.uint8 and 0 <= head_off and head_off + nbytes <= tail_off and tail_off + nbytes <= buffer.numel()
        self.zones = {"head": buffer[head_off:head_off + nbytes], "tail": buffer[tail_off:tail_off + nbytes]}
        self.offsets = {"head": head_off, "tail": tail_off}

    def arm(self) -> None:
        for z in self.zones.values():
            z.fill_(CANARY_VALUE)

    def check(self, what: str = "") -> None:
        for name, z in self.zones.items():
            bad = (z.cpu() != CANARY_VALUE).nonzero()
            if bad.numel():
                first = int(bad[0])
                raise RuntimeError("symmetric workspace%s: %s guard zone overwritten at byte offset %d (value 0x%02x): a peer-memory "
                                   "kernel stored outside its payload region"
                                   % (" (" + what + ")" if what else "", name, self.offsets[name] + first, int(z[first])))

# The workspaces are used through plain peer loads / stores. Binding them to an NVSwitch multicast object is only
# needed by the in-switch (multimem) all-reduce and is therefore opt-in (GV_ENABLE_MULTICAST=1): a process that dies
# while its memory is bound to a multicast object can raise NVLink faults on its peers' GPUs.
if os.environ.get("GV_ENABLE_MULTICAST", "0") != "1":
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")


class GvPeers(ctypes.Structure):
    _fields_ = [("bases", ctypes.c_void_p * 8), ("world", ctypes.c_int), ("rank", ctypes.c_int)]


class FusedGemmArgs(ctypes.Structure):
    _fields_ = [("A", ctypes.c_void_p), ("B", ctypes.c_void_p), ("C", ctypes.c_void_p), ("bias", ctypes.c_void_p),
                ("M", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int),
                ("lda", ctypes.c_int), ("ldb", ctypes.c_int), ("ldc", ctypes.c_int),
                ("a_mode", ctypes.c_int), ("c_mode", ctypes.c_int),
                ("a_off", ctypes.c_longlong), ("c_off", ctypes.c_longlong),
                ("slot_in", ctypes.c_int), ("slot_out", ctypes.c_int), ("epoch", ctypes.c_uint),
                ("gather_buf", ctypes.c_void_p), ("gather_ctr", ctypes.c_void_p)]


def ranks_on_one_node(ranks) -> bool:
    """Whether all ``ranks`` run on one node. Peer-mapped memory only exists inside a node, so a group that spans nodes
    stays on the library collectives. Ranks are numbered node by node (``LOCAL_WORLD_SIZE`` per node, as the launcher sets
    it); without that variable the job is taken to be a single node."""
    try:
        per_node = int(os.environ.get("LOCAL_WORLD_SIZE", "0") or 0)
    except ValueError:
        per_node = 0
    return per_node <= 0 or len({int(r) // per_node for r in ranks}) <= 1


def available(group: Optional[CommGroup]) -> bool:
    if group is None or group.size < 2 or group.size > MAX_RANKS or not torch.cuda.is_available():
        return False
    if not ranks_on_one_node(group.ranks):
        return False
    try:
        import importlib

        importlib.import_module("torch.distributed._symmetric_memory")
        return True
    except Exception:
        return False


class SymmWorkspace:
    def __init__(self, group: CommGroup, payload_bytes: int, device=None):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group
        self.world = group.size
        self.rank = group.rank_in_group(dist.get_rank())
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.canary = None
        guard = 2 * CANARY_BYTES if canaries_enabled() else 0
        self.nbytes = FLAG_BYTES + guard + ((payload_bytes + 255) // 256) * 256
        name = group.group.group_name
        if hasattr(symm_mem, "enable_symm_mem_for_group"):
            try:
                symm_mem.enable_symm_mem_for_group(name)
            except Exception:
                pass
        self.buffer = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=self.device)
        self.handle = symm_mem.rendezvous(self.buffer, group=name)
        self.buffer.zero_()
        torch.cuda.synchronize()
        dist.barrier(group=group.group)
        ptrs = list(self.handle.buffer_ptrs)
        # multicast (NVSwitch) mapping of the same buffer, 0 where the fabric or the driver offers none
        self.multicast_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        self.peers = GvPeers()
        for r in range(8):
            self.peers.bases[r] = ptrs[r] if r < self.world else None
        self.peers.world, self.peers.rank = self.world, self.rank
        self._epoch: Dict[int, int] = {}
        self._bump = FLAG_BYTES
        self._limit = self.nbytes
        if guard:
            # payload regions live between the two guard zones (same offsets on every rank)
            self.canary = CanaryGuard(self.buffer, FLAG_BYTES, self.nbytes - CANARY_BYTES)
            self.canary.arm()
            torch.cuda.synchronize()
            dist.barrier(group=group.group)
            self._bump = FLAG_BYTES + CANARY_BYTES
            self._limit = self.nbytes - CANARY_BYTES
        self._regions: Dict[str, tuple] = {}

    # ------------------------------------------------------------------ regions
    def region(self, name: str, nbytes: int) -> int:
        """Byte offset of a named payload region (allocated on first use; same offset on every rank)."""
        if name in self._regions:
            off, size = self._regions[name]
            if size >= nbytes:
                return off
            raise RuntimeError("symmetric region %r was created with %d bytes, %d requested" % (name, size, nbytes))
        off = self._bump
        size = (nbytes + 255) // 256 * 256
        if off + size > self._limit:
            raise RuntimeError("symmetric workspace exhausted (%d of %d bytes used, %d more requested)" % (off, self._limit, size))
        self._bump = off + size
        self._regions[name] = (off, size)
        return off

    def view(self, off: int, shape, dtype=torch.bfloat16) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty(0, dtype=dtype).element_size()
        return self.buffer[off:off + nbytes].view(dtype).view(*shape)

    def next_epoch(self, slot: int) -> int:
        e = self._epoch.get(slot, 0) + 1
        self._epoch[slot] = e
        return e

    # ------------------------------------------------------------------ primitives
    def barrier(self, slot: int = 15, timeout_ms: int = 0) -> None:
        e = self.next_epoch(slot)
        _lib.check(_lib.lib().gv_comm_barrier(ctypes.byref(self.peers), slot, ctypes.c_uint(e), timeout_ms,
                                              ctypes.c_void_p(_lib.stream_ptr())), "gv_comm_barrier")

    def signal(self, slot: int, epoch: Optional[int] = None) -> int:
        e = self.next_epoch(slot) if epoch is None else epoch
        _lib.check(_lib.lib().gv_comm_signal(ctypes.byref(self.peers), slot, ctypes.c_uint(e),
                                             ctypes.c_void_p(_lib.stream_ptr())), "gv_comm_signal")
        return e

    def wait(self, slot: int, src: int, epoch: int, timeout_ms: int = 0) -> None:
        _lib.check(_lib.lib().gv_comm_wait(ctypes.byref(self.peers), slot, src, ctypes.c_uint(epoch), timeout_ms,
                                           ctypes.c_void_p(_lib.stream_ptr())), "gv_comm_wait")


_WORKSPACES: Dict[tuple, SymmWorkspace] = {}


def workspace(group: CommGroup, payload_bytes: int, tag: str = "act") -> SymmWorkspace:
    """One cached workspace per (group, tag); the first request fixes its size. Creating one is a collective with a
    device synchronisation and a barrier, so a training run creates its workspaces during the first step (one per
    distinct activation shape) and reuses them afterwards; ``workspace_stats`` shows what is held and
    ``release_workspaces`` gives it back."""
    key = (tuple(group.ranks), tag)
    ws = _WORKSPACES.get(key)
    if ws is None:
        ws = SymmWorkspace(group, payload_bytes)
        _WORKSPACES[key] = ws
    return ws


def check_canaries(what: str = "") -> int:
    """Debug mode: verify the guard zones of every cached workspace (synchronises the device; raises on the first
    overwritten byte). Returns the number of workspaces checked (0 when the mode is off)."""
    if not canaries_enabled():
        return 0
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    n = 0
    for key, ws in list(_WORKSPACES.items()):
        if getattr(ws, "canary", None) is not None:
            ws.canary.check(what or key[1])
            n += 1
    return n


def workspace_stats() -> Dict[str, int]:
    """Number of cached workspaces and the bytes of peer-mapped memory they hold on this rank."""
    return {"count": len(_WORKSPACES), "bytes": sum(ws.nbytes for ws in _WORKSPACES.values())}


def release_workspaces(group: Optional[CommGroup] = None, tag_prefix: str = "") -> int:
    """Drop cached workspaces (all of them, or those of one group and / or whose tag starts with ``tag_prefix``) and
    return the bytes released on this rank. Collective in effect: the peers map this rank's buffer, so every rank of
    the affected groups has to call it at the same point of the program, with no kernel on those buffers in flight
    (the call synchronises the device first). Objects that hold a workspace themselves (ZeRO buckets, mailboxes) keep
    theirs alive; what is freed here are the per-shape activation workspaces of the fused tensor-parallel paths, e.g.
    after a change of sequence length or batch size made the old shapes useless."""
    keys = [k for k in _WORKSPACES if (group is None or k[0] == tuple(group.ranks)) and k[1].startswith(tag_prefix)]
    if not keys:
        return 0
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    freed = 0
    for k in keys:
        freed += _WORKSPACES.pop(k).nbytes
    return freed
