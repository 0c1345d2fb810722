"""Host wrapper of the tcgen05 flash-attention kernels (csrc/attention_sm100.cu)."""
from __future__ import annotations

import ctypes

import torch

from . import _lib


def supported(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> bool:
    dh = q.shape[-1]
    if dh % 8 != 0 or dh > 128:
        return False
    for t in (q, k, v):
        if t.dtype != torch.bfloat16 or t.stride(-1) != 1 or t.data_ptr() % 16 != 0:
            return False
        if any(s % 8 for s in t.stride()[:-1]):
            return False
    return q.shape[2] % k.shape[2] == 0


def _strides(t):
    return t.stride(0), t.stride(1), t.stride(2)


_READY = False


def _setup():
    global _READY
    lib = _lib.lib()
    if not _READY:
        cdll = object.__getattribute__(lib, "_cdll")
        cdll.gv_attn_fwd.argtypes = [ctypes.POINTER(_lib.AttnArgs), ctypes.c_void_p]
        cdll.gv_attn_fwd.restype = ctypes.c_int
        cdll.gv_attn_bwd.argtypes = [ctypes.POINTER(_lib.AttnArgs), ctypes.c_void_p]
        cdll.gv_attn_bwd.restype = ctypes.c_int
        _READY = True
    return lib


def _lens(kv_lens, b: int, device):
    if kv_lens is None:
        return None
    t = kv_lens.to(device=device, dtype=torch.int32).contiguous()
    assert t.numel() == b, "kv_lens needs one entry per batch element"
    return t


def _set_dropout(a, dropout) -> None:
    """``dropout`` = (p, seed, head_offset) or None."""
    if dropout is not None and dropout[0] > 0.0:
        a.dropout_p, a.dropout_seed, a.dropout_head_offset = float(dropout[0]), int(dropout[1]) & 0xFFFFFFFFFFFFFFFF, int(dropout[2])


def additive_ld(sq: int, sk: int) -> int:
    """Row stride of every additive-term tensor: a multiple of 64 that covers both sequence lengths."""
    return (max(sq, sk) + 63) // 64 * 64


def pad_rows(t: torch.Tensor, ld: int, dtype, fill=0) -> torch.Tensor:
    """[..., n] -> contiguous [..., ld] of ``dtype`` with the tail filled: the layout the kernels read bias (bf16), additive
    masks (fp32) and group ids (int32, fill -1) in."""
    out = torch.full(tuple(t.shape[:-1]) + (ld,), fill, dtype=dtype, device=t.device)
    out[..., :t.shape[-1]] = t
    return out


class Additive:
    """Score terms of one attention call, in kernel layout (see ``gv_attn_args`` in csrc/include/gv_kernels.h).

    ``bias`` [hq, sq, sk]: additive, shared by the batch (its transpose is kept for the backward kernel);
    ``mask`` [n, sq, sk]: additive, batch element i uses mask[i % n] (general path);
    ``ids`` [n, s] integer group ids (sq == sk): key j is visible to query i iff ids[i] == ids[j]."""

    def __init__(self, sq: int, sk: int, bias=None, mask=None, ids=None):
        self.sq, self.sk, self.ld = sq, sk, additive_ld(sq, sk)
        self.bias = self.bias_t = self.mask = self.ids = None
        if bias is not None:
            assert bias.shape[1:] == (sq, sk)
            self.bias = pad_rows(bias.detach(), self.ld, torch.bfloat16)
            self.bias_t = pad_rows(bias.detach().transpose(1, 2), self.ld, torch.bfloat16)
        if mask is not None:
            assert mask.shape[1:] == (sq, sk)
            self.mask = pad_rows(mask, self.ld, torch.float32)
        if ids is not None:
            assert sq == sk and ids.shape[1] == sq
            self.ids = pad_rows(ids, self.ld, torch.int32, fill=-1)
        assert self.mask is None or self.ids is None or self.mask.shape[0] == self.ids.shape[0]

    def apply(self, a, hq: int) -> None:
        a.bias_ld = self.ld
        if self.bias is not None:
            assert self.bias.shape[0] == hq, "one bias matrix per query head"
            a.bias, a.bias_t = self.bias.data_ptr(), self.bias_t.data_ptr()
        if self.mask is not None:
            a.mask, a.mask_n = self.mask.data_ptr(), self.mask.shape[0]
        if self.ids is not None:
            a.ids, a.mask_n = self.ids.data_ptr(), self.ids.shape[0]


def fwd(q, k, v, causal: bool, scale: float, out=None, kv_lens=None, dropout=None, additive: Additive | None = None):
    lib = _setup()
    b, sq, hq, dh = q.shape
    sk, hk = k.shape[1], k.shape[2]
    o = out if out is not None else torch.empty((b, sq, hq, dh), dtype=q.dtype, device=q.device)
    lse = torch.empty((b, hq, sq), dtype=torch.float32, device=q.device)
    a = _lib.AttnArgs(q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), o=o.data_ptr(), lse=lse.data_ptr(),
                      b=b, sq=sq, sk=sk, hq=hq, hk=hk, dh=dh, causal=int(causal), scale=float(scale))
    lens = _lens(kv_lens, b, q.device)
    a.kv_lens = _lib.p(lens) or None
    _set_dropout(a, dropout)
    if additive is not None:
        additive.apply(a, hq)
    (a.q_stride_b, a.q_stride_s, a.q_stride_h) = _strides(q)
    (a.k_stride_b, a.k_stride_s, a.k_stride_h) = _strides(k)
    (a.v_stride_b, a.v_stride_s, a.v_stride_h) = _strides(v)
    (a.o_stride_b, a.o_stride_s, a.o_stride_h) = _strides(o)
    _lib.check(lib.gv_attn_fwd(a, _lib.stream_ptr()), "gv_attn_fwd")
    return o, lse


def bwd(dout, q, k, v, o, lse, causal: bool, scale: float, dq=None, dk=None, dv=None, kv_lens=None, dq_rope=None,
        dropout=None, additive: Additive | None = None, dbias=None):
    """``dq_rope`` = (inv_freq fp32 [dh / 2], positions int32 [sq * b] in sequence-major token order or None, offset):
    the query gradient leaves the kernel with the inverse rotary rotation already applied. ``additive`` as in ``fwd``;
    ``dbias`` (fp32 zeros [hq, sq, additive.ld]) receives the bias gradient summed over the batch."""
    lib = _setup()
    b, sq, hq, dh = q.shape
    sk, hk = k.shape[1], k.shape[2]
    if dout.stride(-1) != 1 or any(s % 8 for s in dout.stride()[:-1]) or dout.data_ptr() % 16:
        dout = dout.contiguous()
    if dq is None:
        dq = torch.empty((b, sq, hq, dh), dtype=q.dtype, device=q.device)
        dk = torch.empty((b, sk, hk, dh), dtype=q.dtype, device=q.device)
        dv = torch.empty((b, sk, hk, dh), dtype=q.dtype, device=q.device)
    dq_accum = torch.empty((b, sq, hq, dh), dtype=torch.float32, device=q.device)
    delta = torch.empty((b, hq, sq), dtype=torch.float32, device=q.device)
    a = _lib.AttnArgs(q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), o=o.data_ptr(), lse=lse.data_ptr(),
                      dout=dout.data_ptr(), dq=dq.data_ptr(), dk=dk.data_ptr(), dv=dv.data_ptr(),
                      dq_accum=dq_accum.data_ptr(), delta=delta.data_ptr(),
                      b=b, sq=sq, sk=sk, hq=hq, hk=hk, dh=dh, causal=int(causal), scale=float(scale))
    lens = _lens(kv_lens, b, q.device)
    a.kv_lens = _lib.p(lens) or None
    (a.q_stride_b, a.q_stride_s, a.q_stride_h) = _strides(q)
    (a.k_stride_b, a.k_stride_s, a.k_stride_h) = _strides(k)
    (a.v_stride_b, a.v_stride_s, a.v_stride_h) = _strides(v)
    (a.o_stride_b, a.o_stride_s, a.o_stride_h) = _strides(o)
    _set_dropout(a, dropout)
    if additive is not None:
        additive.apply(a, hq)
    if dbias is not None:
        assert additive is not None and additive.bias is not None and dbias.shape == additive.bias.shape
        assert dbias.dtype == torch.float32 and dbias.is_contiguous()
        a.dbias = dbias.data_ptr()
    if dq_rope is not None:
        inv_freq, pos, off = dq_rope
        pos = None if pos is None else pos.to(device=q.device, dtype=torch.int32).contiguous()
        a.dq_rope_inv_freq, a.dq_rope_pos, a.dq_rope_pos_offset = inv_freq.data_ptr(), (_lib.p(pos) or None), int(off)
    (a.do_stride_b, a.do_stride_s, a.do_stride_h) = _strides(dout)
    (a.dq_stride_b, a.dq_stride_s, a.dq_stride_h) = _strides(dq)
    (a.dk_stride_b, a.dk_stride_s, a.dk_stride_h) = _strides(dk)
    (a.dv_stride_b, a.dv_stride_s, a.dv_stride_h) = _strides(dv)
    _lib.check(lib.gv_attn_bwd(a, _lib.stream_ptr()), "gv_attn_bwd")
    return dq, dk, dv
