"""Low-level (non-autograd) operator wrappers.

bf16 CUDA tensors run the hand-written sm_100a kernels of ``csrc/``; CPU tensors and fp32/fp16
tensors run an equivalent PyTorch expression (used by the gloo plumbing tests and as the numerical
oracle of the GPU tests). Function names mirror csrc/include/gv_kernels.h.
"""
from __future__ import annotations

import math
from ctypes import c_void_p

import torch
import torch.nn.functional as F

from . import _lib

_f = float


def _native(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16


def _vp(t):
    return c_void_p(0 if t is None else t.data_ptr())


def _s():
    return c_void_p(_lib.stream_ptr())


# ----------------------------------------------------------------------------- normalisation
def _norm_scratch(rows: int, cols: int, layer: int, device) -> torch.Tensor:
    """Partial weight-gradient rows of the two-stage (atomic-free, bitwise repeatable) norm backward: one per CTA."""
    fn = _lib.lib().gv_norm_bwd_scratch_elems
    raw = getattr(fn, "raw", fn)
    raw.restype = _lib.c_longlong
    n = int(raw(int(rows), int(cols), int(layer)))
    return torch.empty(max(n, 1), dtype=torch.float32, device=device)


def rmsnorm_fwd(x: torch.Tensor, w: torch.Tensor, eps: float, residual: torch.Tensor | None = None):
    """Returns (y, h, rstd) with h = x + residual (h is x itself when residual is None)."""
    rows, cols = x.numel() // x.shape[-1], x.shape[-1]
    if _native(x) and cols % 8 == 0 and cols <= 8192:
        x = x.contiguous()
        y = torch.empty_like(x)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        h = torch.empty_like(x) if residual is not None else x
        if residual is not None:
            residual = residual.contiguous()
        rc = _lib.lib().gv_rmsnorm_fwd(_vp(x), _vp(residual), _vp(w), _vp(y), _vp(h if residual is not None else None),
                                       _vp(rstd), rows, cols, _lib.c_float(eps), _s())
        _lib.check(rc, "gv_rmsnorm_fwd")
        return y, h, rstd
    h = x if residual is None else (x + residual)
    hf = h.float()
    rstd = torch.rsqrt(hf.pow(2).mean(-1) + eps)
    y = (hf * rstd.unsqueeze(-1) * w.float()).to(x.dtype)
    return y, h, rstd.reshape(-1)


def rmsnorm_bwd(dy, h, w, rstd, dres=None, dw_accum: torch.Tensor | None = None):
    """Returns dx (= grad wrt h, plus dres). The weight gradient is added to fp32 ``dw_accum``."""
    rows, cols = h.numel() // h.shape[-1], h.shape[-1]
    if _native(h) and cols % 8 == 0 and cols <= 8192 and dw_accum is not None and dw_accum.dtype == torch.float32:
        dy = dy.contiguous()
        dx = torch.empty_like(h)
        if dres is not None:
            dres = dres.contiguous()
        scratch = _norm_scratch(rows, cols, 0, h.device)
        rc = _lib.lib().gv_rmsnorm_bwd(_vp(dy), _vp(h), _vp(w), _vp(rstd), _vp(dres), _vp(dx), _vp(dw_accum), _vp(scratch),
                                       _lib.c_longlong(scratch.numel()), rows, cols, _s())
        _lib.check(rc, "gv_rmsnorm_bwd")
        return dx
    hf = h.float().reshape(rows, cols)
    dyf = dy.float().reshape(rows, cols)
    r = rstd.reshape(rows, 1).float()
    xh = hf * r
    g = dyf * w.float()
    dx = r * (g - xh * (g * xh).mean(-1, keepdim=True))
    if dres is not None:
        dx = dx + dres.float().reshape(rows, cols)
    if dw_accum is not None:
        dw_accum.add_((dyf * xh).sum(0).to(dw_accum.dtype))
    return dx.to(h.dtype).reshape(h.shape)


def layernorm_fwd(x, w, b, eps, residual=None):
    """Returns (y, h, mean, rstd)."""
    rows, cols = x.numel() // x.shape[-1], x.shape[-1]
    if _native(x) and cols % 8 == 0 and cols <= 8192:
        x = x.contiguous()
        y = torch.empty_like(x)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        h = torch.empty_like(x) if residual is not None else x
        if residual is not None:
            residual = residual.contiguous()
        rc = _lib.lib().gv_layernorm_fwd(_vp(x), _vp(residual), _vp(w), _vp(b), _vp(y),
                                         _vp(h if residual is not None else None), _vp(mean), _vp(rstd), rows, cols,
                                         _lib.c_float(eps), _s())
        _lib.check(rc, "gv_layernorm_fwd")
        return y, h, mean, rstd
    h = x if residual is None else (x + residual)
    hf = h.float()
    mean = hf.mean(-1)
    var = hf.var(-1, unbiased=False)
    rstd = torch.rsqrt(var + eps)
    y = ((hf - mean.unsqueeze(-1)) * rstd.unsqueeze(-1) * w.float() + b.float()).to(x.dtype)
    return y, h, mean.reshape(-1), rstd.reshape(-1)


def layernorm_bwd(dy, h, w, mean, rstd, dres=None, dw_accum=None, db_accum=None):
    rows, cols = h.numel() // h.shape[-1], h.shape[-1]
    if (_native(h) and cols % 8 == 0 and cols <= 8192 and dw_accum is not None and dw_accum.dtype == torch.float32
            and db_accum is not None and db_accum.dtype == torch.float32):
        dy = dy.contiguous()
        dx = torch.empty_like(h)
        if dres is not None:
            dres = dres.contiguous()
        scratch = _norm_scratch(rows, cols, 1, h.device)
        rc = _lib.lib().gv_layernorm_bwd(_vp(dy), _vp(h), _vp(w), _vp(mean), _vp(rstd), _vp(dres), _vp(dx),
                                         _vp(dw_accum), _vp(db_accum), _vp(scratch), _lib.c_longlong(scratch.numel()),
                                         rows, cols, _s())
        _lib.check(rc, "gv_layernorm_bwd")
        return dx
    hf = h.float().reshape(rows, cols)
    dyf = dy.float().reshape(rows, cols)
    r = rstd.reshape(rows, 1).float()
    xh = (hf - mean.reshape(rows, 1).float()) * r
    g = dyf * w.float()
    dx = r * (g - g.mean(-1, keepdim=True) - xh * (g * xh).mean(-1, keepdim=True))
    if dres is not None:
        dx = dx + dres.float().reshape(rows, cols)
    if dw_accum is not None:
        dw_accum.add_((dyf * xh).sum(0).to(dw_accum.dtype))
    if db_accum is not None:
        db_accum.add_(dyf.sum(0).to(db_accum.dtype))
    return dx.to(h.dtype).reshape(h.shape)


# ----------------------------------------------------------------------------- RoPE
def rope_inv_freq(dh: int, base: float, device) -> torch.Tensor:
    return 1.0 / (base ** (torch.arange(0, dh, 2, dtype=torch.float32, device=device) / dh))


def rope_(x: torch.Tensor, inv_freq: torch.Tensor, pos_div: int = 1, pos_mod: int = 0, pos_offset: int = 0,
          positions: torch.Tensor | None = None, inverse: bool = False) -> torch.Tensor:
    """In-place rotary embedding on ``x`` = [tokens, heads, dh] (a strided view is fine: token stride
    arbitrary, head stride dh, unit inner stride). Token t has position ``positions[t]`` or
    ``(t // pos_div) % pos_mod + pos_offset`` (``pos_mod`` 0 = no wrap): batch-major tokens use
    ``pos_div=1, pos_mod=seq``; sequence-major tokens use ``pos_div=batch``. ``inverse`` applies the
    transposed rotation (the backward)."""
    tokens, heads, dh = x.shape
    if (_native(x) and dh % 16 == 0 and x.stride(2) == 1 and x.stride(1) == dh and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0):
        pos32 = None
        if positions is not None:
            pos32 = positions.to(torch.int32).contiguous()
        rc = _lib.lib().gv_rope(_vp(x), _vp(pos32), _vp(inv_freq), _lib.c_longlong(tokens), heads, dh,
                                _lib.c_longlong(x.stride(0)), int(pos_div), int(pos_mod), int(pos_offset), int(inverse),
                                _s())
        _lib.check(rc, "gv_rope")
        return x
    if positions is None:
        positions = torch.arange(tokens, device=x.device) // max(pos_div, 1)
        if pos_mod:
            positions = positions % pos_mod
        positions = positions + pos_offset
    ang = positions.float().unsqueeze(-1) * inv_freq.float().unsqueeze(0)  # [tokens, dh/2]
    cos, sin = ang.cos().unsqueeze(1), ang.sin().unsqueeze(1)
    if inverse:
        sin = -sin
    xf = x.float()
    a, b = xf[..., : dh // 2], xf[..., dh // 2:]
    out = torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)
    x.copy_(out.to(x.dtype))
    return x


# ----------------------------------------------------------------------------- activations
def swiglu_fwd(gu: torch.Tensor) -> torch.Tensor:
    f = gu.shape[-1] // 2
    rows = gu.numel() // gu.shape[-1]
    if _native(gu) and f % 8 == 0 and gu.is_contiguous():
        out = torch.empty(*gu.shape[:-1], f, dtype=gu.dtype, device=gu.device)
        _lib.check(_lib.lib().gv_swiglu_fwd(_vp(gu), _vp(out), _lib.c_longlong(rows), f, _s()), "gv_swiglu_fwd")
        return out
    g, u = gu.float().chunk(2, dim=-1)
    return (F.silu(g) * u).to(gu.dtype)


def swiglu_bwd(dout: torch.Tensor, gu: torch.Tensor) -> torch.Tensor:
    f = gu.shape[-1] // 2
    rows = gu.numel() // gu.shape[-1]
    if _native(gu) and f % 8 == 0 and gu.is_contiguous():
        dout = dout.contiguous()
        dgu = torch.empty_like(gu)
        _lib.check(_lib.lib().gv_swiglu_bwd(_vp(dout), _vp(gu), _vp(dgu), _lib.c_longlong(rows), f, _s()),
                   "gv_swiglu_bwd")
        return dgu
    g, u = gu.float().chunk(2, dim=-1)
    d = dout.float()
    sg = torch.sigmoid(g)
    silu = g * sg
    return torch.cat([d * u * (sg + silu * (1 - sg)), d * silu], dim=-1).to(gu.dtype)


def gelu_fwd(x: torch.Tensor) -> torch.Tensor:
    if _native(x) and x.numel() % 8 == 0 and x.is_contiguous():
        y = torch.empty_like(x)
        _lib.check(_lib.lib().gv_gelu_fwd(_vp(x), _vp(y), _lib.c_longlong(x.numel()), _s()), "gv_gelu_fwd")
        return y
    return F.gelu(x.float(), approximate="tanh").to(x.dtype)


def gelu_bwd(dy: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    if _native(x) and x.numel() % 8 == 0 and x.is_contiguous():
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        _lib.check(_lib.lib().gv_gelu_bwd(_vp(dy), _vp(x), _vp(dx), _lib.c_longlong(x.numel()), _s()), "gv_gelu_bwd")
        return dx
    xf = x.float()
    k0, k1 = 0.7978845608028654, 0.044715
    t = torch.tanh(k0 * (xf + k1 * xf ** 3))
    g = 0.5 * (1 + t) + 0.5 * xf * (1 - t * t) * k0 * (1 + 3 * k1 * xf * xf)
    return (dy.float() * g).to(x.dtype)


def colsum_accum(dy: torch.Tensor, out: torch.Tensor) -> None:
    """out[c] += sum_r dy[r, c] (bias gradient)."""
    cols = dy.shape[-1]
    rows = dy.numel() // cols
    if _native(dy) and cols % 8 == 0 and out.dtype == torch.float32 and dy.is_contiguous():
        _lib.check(_lib.lib().gv_colsum_accum(_vp(dy), _vp(out), _lib.c_longlong(rows), cols, _s()), "gv_colsum_accum")
        return
    out.add_(dy.float().reshape(rows, cols).sum(0).to(out.dtype))


# ----------------------------------------------------------------------------- embedding
def embedding_fwd(ids: torch.Tensor, table: torch.Tensor, vocab_start: int = 0,
                  pos_ids: torch.Tensor | None = None, pos_table: torch.Tensor | None = None) -> torch.Tensor:
    """out[t] = table[ids[t]-vocab_start] (zero outside this vocab shard) (+ pos_table[pos_ids[t]])."""
    hidden = table.shape[1]
    flat = ids.reshape(-1)
    if _native(table) and hidden % 8 == 0:
        flat = flat.to(torch.int64).contiguous()
        out = torch.empty(flat.numel(), hidden, dtype=table.dtype, device=table.device)
        p32 = pos_ids.reshape(-1).to(torch.int32).contiguous() if pos_table is not None else None
        rc = _lib.lib().gv_embedding_fwd(_vp(flat), _vp(table), _vp(p32), _vp(pos_table), _vp(out),
                                         _lib.c_longlong(flat.numel()), hidden, _lib.c_longlong(vocab_start),
                                         _lib.c_longlong(table.shape[0]), _s())
        _lib.check(rc, "gv_embedding_fwd")
        return out.reshape(*ids.shape, hidden)
    local = flat - vocab_start
    mask = (local >= 0) & (local < table.shape[0])
    out = table[local.clamp(0, table.shape[0] - 1)] * mask.unsqueeze(-1).to(table.dtype)
    if pos_table is not None:
        out = out + pos_table[pos_ids.reshape(-1)]
    return out.reshape(*ids.shape, hidden)


def embedding_bwd(ids: torch.Tensor, dout: torch.Tensor, dtable_accum: torch.Tensor, vocab_start: int = 0) -> None:
    hidden = dtable_accum.shape[1]
    flat = ids.reshape(-1)
    if _native(dout) and hidden % 8 == 0 and dtable_accum.dtype == torch.float32:
        flat = flat.to(torch.int64).contiguous()
        dout = dout.contiguous()
        rc = _lib.lib().gv_embedding_bwd(_vp(flat), _vp(dout), _vp(dtable_accum), _lib.c_longlong(flat.numel()), hidden,
                                         _lib.c_longlong(vocab_start), _lib.c_longlong(dtable_accum.shape[0]), _s())
        _lib.check(rc, "gv_embedding_bwd")
        return
    local = flat - vocab_start
    mask = (local >= 0) & (local < dtable_accum.shape[0])
    d = dout.reshape(-1, hidden)[mask].to(dtable_accum.dtype)
    dtable_accum.index_add_(0, local[mask], d)


# ----------------------------------------------------------------------------- cross entropy
def xent_stats(logits: torch.Tensor, labels: torch.Tensor, vocab_start: int = 0):
    """Per-row (max, sum exp(x - max), target logit or 0) over this rank's vocab shard."""
    rows, v = logits.shape
    if _native(logits) and logits.stride(1) == 1 and logits.stride(0) % 8 == 0:
        labels = labels.reshape(-1).to(torch.int64).contiguous()
        mx = torch.empty(rows, dtype=torch.float32, device=logits.device)
        se = torch.empty_like(mx)
        tg = torch.empty_like(mx)
        rc = _lib.lib().gv_xent_stats(_vp(logits), _vp(labels), _vp(mx), _vp(se), _vp(tg), _lib.c_longlong(rows), v,
                                      _lib.c_longlong(logits.stride(0)), _lib.c_longlong(vocab_start), _s())
        _lib.check(rc, "gv_xent_stats")
        return mx, se, tg
    lf = logits.float()
    mx = lf.max(-1).values
    se = (lf - mx.unsqueeze(-1)).exp().sum(-1)
    local = labels.reshape(-1) - vocab_start
    inside = (local >= 0) & (local < v)
    tg = lf.gather(1, local.clamp(0, v - 1).unsqueeze(1)).squeeze(1) * inside.float()
    return mx, se, tg


def xent_loss_grad_(logits: torch.Tensor, labels: torch.Tensor, mx, se, tg, grad_scale: float, vocab_start: int = 0,
                    ignore_index: int = -100, scale_tensor: torch.Tensor | None = None) -> torch.Tensor:
    """Given the (cross-shard reduced) statistics, returns per-row loss and overwrites ``logits`` with
    (softmax - onehot) * grad_scale * scale_tensor[row] (``scale_tensor``: optional fp32 per-row upstream
    gradient)."""
    rows, v = logits.shape
    labels = labels.reshape(-1)
    if _native(logits) and logits.stride(1) == 1 and logits.stride(0) % 8 == 0:
        labels = labels.to(torch.int64).contiguous()
        loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
        rc = _lib.lib().gv_xent_loss_grad(_vp(logits), _vp(labels), _vp(mx), _vp(se), _vp(tg), _vp(loss),
                                          _lib.c_float(grad_scale), _vp(scale_tensor), _lib.c_longlong(rows), v,
                                          _lib.c_longlong(logits.stride(0)), _lib.c_longlong(vocab_start),
                                          _lib.c_longlong(ignore_index), _s())
        _lib.check(rc, "gv_xent_loss_grad")
        return loss
    lf = logits.float()
    keep = (labels != ignore_index).float()
    loss = (se.log() + mx - tg) * keep
    prob = (lf - mx.unsqueeze(-1)).exp() / se.unsqueeze(-1)
    local = labels - vocab_start
    inside = (local >= 0) & (local < v) & (labels != ignore_index)
    onehot = torch.zeros_like(prob)
    onehot[inside, local[inside]] = 1.0
    gs = keep * grad_scale
    if scale_tensor is not None:
        gs = gs * scale_tensor.float().reshape(-1)
    logits.copy_(((prob - onehot) * gs.unsqueeze(-1)).to(logits.dtype))
    return loss


# ----------------------------------------------------------------------------- optimizer
def adamw_step_(master, m, v, grad, param, *, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0,
                clip_coef: torch.Tensor | None = None) -> None:
    """Fused AdamW on flat buffers: fp32 master / m / v, fp32 or bf16 grad, optional low-precision param copy."""
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    n = master.numel()
    if master.is_cuda and master.dtype == torch.float32 and grad.dtype in (torch.float32, torch.bfloat16) and \
            (param is None or param.dtype == torch.bfloat16):
        rc = _lib.lib().gv_adamw(_vp(master), _vp(m), _vp(v), _vp(grad), int(grad.dtype == torch.bfloat16), _vp(param),
                                 _lib.c_longlong(n), _lib.c_float(lr), _lib.c_float(beta1), _lib.c_float(beta2),
                                 _lib.c_float(eps), _lib.c_float(weight_decay), _lib.c_float(bc1), _lib.c_float(bc2),
                                 _lib.c_float(grad_scale), _vp(clip_coef), _s())
        _lib.check(rc, "gv_adamw")
        return
    g = grad.to(master.dtype) * grad_scale
    if clip_coef is not None:
        g = g * clip_coef.to(master.dtype)
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    upd = (m / bc1) / ((v / bc2).sqrt() + eps) + weight_decay * master
    master.add_(upd, alpha=-lr)
    if param is not None:
        param.copy_(master)


def sumsq_accum(x: torch.Tensor, out: torch.Tensor) -> None:
    """out[0] += sum(x^2) (fp32)."""
    if x.is_cuda and x.dtype in (torch.float32, torch.bfloat16) and x.is_contiguous() and out.dtype == torch.float32:
        rc = _lib.lib().gv_sumsq_accum(_vp(x), int(x.dtype == torch.bfloat16), _lib.c_longlong(x.numel()), _vp(out), _s())
        _lib.check(rc, "gv_sumsq_accum")
        return
    out.add_(x.float().pow(2).sum().to(out.dtype))


def lse_merge_(acc: torch.Tensor, lse_acc: torch.Tensor, o_blk: torch.Tensor, lse_blk: torch.Tensor, s_off: int = 0) -> None:
    """Fold a partial attention result (o_blk [b, sb, h, dh], lse_blk [b, h, sb]) over query rows [s_off, s_off + sb)
    into the fp32 accumulators acc [b, s, h, dh] / lse_acc [b, h, s] (reference: the TorchScript merge of the zigzag
    ring attention, galvatron/core/runtime/tensor_parallel/transformer.py:2208-2249)."""
    b, s, h, dh = acc.shape
    sb = o_blk.shape[1]
    if (acc.is_cuda and acc.dtype == torch.float32 and acc.is_contiguous() and lse_acc.is_contiguous()
            and o_blk.dtype == torch.bfloat16 and o_blk.stride(-1) == 1 and lse_blk.dtype == torch.float32):
        lse_blk = lse_blk.contiguous()
        rc = _lib.lib().gv_lse_merge(_vp(acc), _vp(lse_acc), _vp(o_blk), _vp(lse_blk), b, s, sb, s_off, h, dh,
                                     _lib.c_longlong(o_blk.stride(0)), _lib.c_longlong(o_blk.stride(1)),
                                     _lib.c_longlong(o_blk.stride(2)), _s())
        _lib.check(rc, "gv_lse_merge")
        return
    la = lse_acc[:, :, s_off:s_off + sb]
    lb = lse_blk.float()
    ln = torch.logaddexp(la, lb)
    wa = torch.exp(la - ln).nan_to_num(0.0).permute(0, 2, 1).unsqueeze(-1)          # [b, sb, h, 1]
    wb = torch.exp(lb - ln).nan_to_num(0.0).permute(0, 2, 1).unsqueeze(-1)
    a = acc[:, s_off:s_off + sb]
    a.copy_(a * wa + o_blk.float() * wb)
    la.copy_(ln)


# ----------------------------------------------------------------------------- attention
def _key_padding(kv_lens, sk: int, device):
    """[b, 1, 1, sk] bool, True where the key is padding (index >= kv_lens[b])."""
    return (torch.arange(sk, device=device).view(1, 1, 1, sk) >= kv_lens.to(device).view(-1, 1, 1, 1))


def _mix32(x):
    return x & 0xFFFFFFFF


def dropout_keep_mask(p: float, seed: int, b: int, hq: int, sq: int, sk: int, head_offset: int = 0, device="cpu"):
    """[b, hq, sq, sk] bool: which attention probabilities survive dropout. Same counter-based draw as the kernels
    (csrc/attention_sm100.cu ``drop_key`` / ``drop_keep``): a pure function of (seed, batch, head, q, k)."""
    i64 = torch.int64
    seed = int(seed) & 0xFFFFFFFFFFFFFFFF
    x0 = (seed & 0xFFFFFFFF) ^ _mix32((seed >> 32) * 0x9E3779B1)
    bb = torch.arange(b, dtype=i64, device=device).view(b, 1)
    hh = (torch.arange(hq, dtype=i64, device=device) + head_offset).view(1, hq)
    x = x0 ^ _mix32(bb * 0x85EBCA77 + 0x165667B1)
    x = x ^ (x >> 15)
    x = _mix32(x * 0x2C1B3C6D)
    x = x ^ _mix32(hh * 0xC2B2AE3D + 0x27D4EB2F)
    x = x ^ (x >> 13)
    x = _mix32(x * 0x297A2D39)
    key = (x ^ (x >> 16)).view(b, hq, 1, 1)
    qq = torch.arange(sq, dtype=i64, device=device).view(1, 1, sq, 1)
    kk = torch.arange(sk, dtype=i64, device=device).view(1, 1, 1, sk)
    y = key ^ _mix32(qq * 0x9E3779B1) ^ _mix32(kk * 0x85EBCA77)
    y = y ^ (y >> 15)
    y = _mix32(y * 0x2C1B3C6D)
    y = y ^ (y >> 12)
    y = _mix32(y * 0x297A2D39)
    y = y ^ (y >> 15)
    thr = min(int(float(p) * 4294967296.0), 4294967295)
    return y >= max(thr, 1)


def attention_reference(q, k, v, causal: bool, scale: float, kv_lens=None, dropout=None):
    """fp32 attention with log-sum-exp output. q: [b, sq, hq, dh]; k, v: [b, sk, hk, dh]; ``kv_lens`` [b]: number
    of leading keys per batch element that are real (the rest is padding)."""
    b, sq, hq, dh = q.shape
    sk, hk = k.shape[1], k.shape[2]
    rep = hq // hk
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        mask = torch.ones(sq, sk, dtype=torch.bool, device=q.device).tril(diagonal=sk - sq)
        s = s.masked_fill(~mask, float("-inf"))
    if kv_lens is not None:
        s = s.masked_fill(_key_padding(kv_lens, sk, q.device), float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    if dropout is not None and dropout[0] > 0.0:
        keep = dropout_keep_mask(dropout[0], dropout[1], b, hq, sq, sk, dropout[2], q.device)
        p = p * keep.to(p.dtype) / (1.0 - dropout[0])
    o = torch.matmul(p, vf).permute(0, 2, 1, 3)
    return o.to(q.dtype), lse


def biased_attention_reference(q, k, v, scale: float, bias=None, mask=None, ids=None):
    """fp32 attention with additive score terms. q, k, v: [b, s, h, dh]; ``bias`` [h, sq, sk] is shared by the batch,
    ``mask`` [n, sq, sk] (additive) and ``ids`` [n, s] (group ids: a query sees the keys of its own group) belong to batch
    element ``i % n``. Differentiable (plain PyTorch expressions)."""
    b, sq, h, dh = q.shape
    s = torch.matmul(q.float().permute(0, 2, 1, 3), k.float().permute(0, 2, 3, 1)) * scale
    if bias is not None:
        s = s + bias.float().unsqueeze(0)
    if mask is not None:
        n = mask.shape[0]
        s = (s.view(b // n, n, h, sq, -1) + mask.float().view(1, n, 1, sq, -1)).view(b, h, sq, -1)
    if ids is not None:
        n = ids.shape[0]
        hidden = (ids[:, :, None] != ids[:, None, :]).view(1, n, 1, sq, sq)
        s = s.view(b // n, n, h, sq, sq).masked_fill(hidden, float("-inf")).view(b, h, sq, sq)
    p = torch.softmax(s, dim=-1)
    return torch.matmul(p, v.float().permute(0, 2, 1, 3)).permute(0, 2, 1, 3).to(q.dtype)


def biased_attention_native(q, k, v) -> bool:
    """Whether the tcgen05 kernels take these operands for the additive-bias path."""
    from . import attention as _attn

    return _native(q) and _attn.supported(q, k, v)


def _pads_to_native(q) -> bool:
    return q.dtype == torch.bfloat16 and q.shape[-1] % 8 != 0 and q.shape[-1] < 128


def _pad_last(t, dh: int):
    return torch.nn.functional.pad(t, (0, (dh + 7) // 8 * 8 - dh))


def attention_fwd(q, k, v, causal: bool, scale: float | None = None, out: torch.Tensor | None = None, kv_lens=None,
                  dropout=None):
    """Returns (o [b, sq, hq, dh], lse [b, hq, sq] fp32). Strided q/k/v views (e.g. slices of a packed
    QKV projection) are consumed in place; ``out`` may be a strided [b, sq, hq, dh] view to fill."""
    from . import attention as _attn

    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    if _native(q) and _attn.supported(q, k, v):
        return _attn.fwd(q, k, v, causal, scale, out, kv_lens, dropout)
    if _native(q) and _pads_to_native(q):
        # head sizes that are not a multiple of 8 (GPT-2 XL: 50): zero columns change neither the scores nor the output
        dh = q.shape[-1]
        qp, kp, vp = (_pad_last(t, dh) for t in (q, k, v))
        if _attn.supported(qp, kp, vp):
            o, lse = _attn.fwd(qp, kp, vp, causal, scale, None, kv_lens, dropout)
            o = o[..., :dh]
            if out is not None:
                out.copy_(o)
                o = out
            return o, lse
    o, lse = attention_reference(q, k, v, causal, scale, kv_lens, dropout)
    if out is not None:
        out.copy_(o)
        o = out
    return o, lse


def attention_bwd(dout, q, k, v, o, lse, causal: bool, scale: float | None = None, dq=None, dk=None, dv=None, kv_lens=None,
                  dq_rope=None, dropout=None):
    """Returns (dq, dk, dv); pre-allocated (possibly strided) outputs may be passed. ``dq_rope`` (native kernel only,
    see ``ops.attention.bwd``) folds the inverse rotary rotation of dq into the kernel; returns True in 4th place when
    it was applied."""
    from . import attention as _attn

    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    if _native(q) and _attn.supported(q, k, v):
        return _attn.bwd(dout, q, k, v, o, lse, causal, scale, dq, dk, dv, kv_lens, dq_rope, dropout)
    if _native(q) and _pads_to_native(q):
        dh = q.shape[-1]
        qp, kp, vp, op, dop = (_pad_last(t, dh) for t in (q, k, v, o, dout))
        if _attn.supported(qp, kp, vp):
            gq, gk, gv = (g[..., :dh] for g in _attn.bwd(dop, qp, kp, vp, op, lse, causal, scale, None, None, None, kv_lens, None, dropout))
            if dq is not None:
                dq.copy_(gq); dk.copy_(gk); dv.copy_(gv)
                return dq, dk, dv
            return gq, gk, gv
    b, sq, hq, dh = q.shape
    sk, hk = k.shape[1], k.shape[2]
    rep = hq // hk
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    dof = dout.float().permute(0, 2, 1, 3)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        mask = torch.ones(sq, sk, dtype=torch.bool, device=q.device).tril(diagonal=sk - sq)
        s = s.masked_fill(~mask, float("-inf"))
    if kv_lens is not None:
        s = s.masked_fill(_key_padding(kv_lens, sk, q.device), float("-inf"))
    p = torch.exp(s - lse.float().unsqueeze(-1))
    pd = p
    dp = torch.matmul(dof, vf.transpose(-1, -2))
    if dropout is not None and dropout[0] > 0.0:
        keep = dropout_keep_mask(dropout[0], dropout[1], b, hq, sq, sk, dropout[2], q.device).to(p.dtype) / (1.0 - dropout[0])
        pd = p * keep
        dp = dp * keep
    dvf = torch.matmul(pd.transpose(-1, -2), dof)
    delta = (dof * o.float().permute(0, 2, 1, 3)).sum(-1, keepdim=True)
    ds = p * (dp - delta) * scale
    dqf = torch.matmul(ds, kf)
    dkf = torch.matmul(ds.transpose(-1, -2), qf)
    dkf = dkf.reshape(b, hk, rep, sk, dh).sum(2)
    dvf = dvf.reshape(b, hk, rep, sk, dh).sum(2)
    rq, rk, rv = dqf.permute(0, 2, 1, 3).to(q.dtype), dkf.permute(0, 2, 1, 3).to(k.dtype), dvf.permute(0, 2, 1, 3).to(v.dtype)
    if dq is not None:
        dq.copy_(rq); dk.copy_(rk); dv.copy_(rv)
        return dq, dk, dv
    return rq, rk, rv
