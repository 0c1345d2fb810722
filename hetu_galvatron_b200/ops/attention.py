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


def pad_additive(t: torch.Tensor, sk: int) -> torch.Tensor:
    """An additive score term [n, sq, sk] (any float dtype) as the kernels read it: fp32, contiguous, rows padded with zeros to
    a multiple of 64 columns."""
    ld = (sk + 63) // 64 * 64
    out = torch.zeros(t.shape[0], t.shape[1], ld, dtype=torch.float32, device=t.device)
    out[:, :, :sk] = t
    return out


def _set_additive(a, bias, mask, sq: int, sk: int, hq: int) -> None:
    """``bias`` [hq, sq, ld] / ``mask`` [mask_n, sq, ld]: fp32 outputs of ``pad_additive`` (either may be None)."""
    ld = None
    for name, t in (("bias", bias), ("mask", mask)):
        if t is None:
            continue
        assert t.dtype == torch.float32 and t.is_contiguous() and t.shape[1] == sq and t.shape[2] % 64 == 0 and t.shape[2] >= sk, \
            "%s must come from pad_additive" % name
        assert ld in (None, t.shape[2]), "bias and mask need the same row stride"
        ld = t.shape[2]
    if bias is not None:
        assert bias.shape[0] == hq, "one bias matrix per query head"
        a.bias = bias.data_ptr()
    if mask is not None:
        a.mask, a.mask_n = mask.data_ptr(), mask.shape[0]
    if ld is not None:
        a.bias_ld = ld


def fwd(q, k, v, causal: bool, scale: float, out=None, kv_lens=None, dropout=None, bias=None, mask=None):
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
    _set_additive(a, bias, mask, sq, sk, hq)
    (a.q_stride_b, a.q_stride_s, a.q_stride_h) = _strides(q)
    (a.k_stride_b, a.k_stride_s, a.k_stride_h) = _strides(k)
    (a.v_stride_b, a.v_stride_s, a.v_stride_h) = _strides(v)
    (a.o_stride_b, a.o_stride_s, a.o_stride_h) = _strides(o)
    _lib.check(lib.gv_attn_fwd(a, _lib.stream_ptr()), "gv_attn_fwd")
    return o, lse


def bwd(dout, q, k, v, o, lse, causal: bool, scale: float, dq=None, dk=None, dv=None, kv_lens=None, dq_rope=None,
        dropout=None, bias=None, mask=None, dbias=None):
    """``dq_rope`` = (inv_freq fp32 [dh / 2], positions int32 [sq * b] in sequence-major token order or None, offset):
    the query gradient leaves the kernel with the inverse rotary rotation already applied. ``bias`` / ``mask`` as in
    ``fwd``; ``dbias`` (fp32, zeroed, shaped like ``bias``) receives the bias gradient summed over the batch."""
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
    _set_additive(a, bias, mask, sq, sk, hq)
    if dbias is not None:
        assert bias is not None and dbias.shape == bias.shape and dbias.dtype == torch.float32 and dbias.is_contiguous()
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
