"""GEMM entry points over the tcgen05 kernel (csrc/gemm_sm100.cu).

``gemm`` computes ``C[M,N] = alpha * A[M,K] @ B[N,K]^T (+bias) (+residual) (+C)``; either operand
may be handed over in its transposed storage (``a_mn`` / ``b_mn``), which is how the input- and
weight-gradient GEMMs of a linear layer read ``dY``, ``W`` and ``X`` without materialising a
transpose (reference: megatron/core/tensor_parallel/layers.py:417,462,534).
"""
from __future__ import annotations

import torch

from . import _lib


def _use_native(*ts) -> bool:
    t0 = ts[0]
    if not t0.is_cuda:
        return False
    return all(t is None or (t.is_cuda and t.dtype == torch.bfloat16) for t in ts)


def _row_major_2d(t: torch.Tensor) -> torch.Tensor:
    if t.dim() != 2:
        t = t.reshape(-1, t.shape[-1])
    if t.stride(1) != 1 or t.stride(0) % 8 != 0 or t.data_ptr() % 16 != 0:
        t = t.contiguous()
    return t


class RopeEpilogue:
    """Rotary embedding applied by the GEMM epilogue to the first ``cols`` output columns (heads of ``dh`` = 64 or 128
    columns, non-interleaved halves): the position of output row r is ``positions[r]`` (int32) or ``r // pos_div +
    pos_offset``. Saves the separate pass over q and k that follows a packed QKV projection."""

    def __init__(self, cols: int, dh: int, inv_freq: torch.Tensor, positions=None, pos_div: int = 1, pos_offset: int = 0):
        self.cols, self.dh, self.inv_freq = int(cols), int(dh), inv_freq
        self.positions = None if positions is None else positions.to(torch.int32).contiguous()
        self.pos_div, self.pos_offset = int(pos_div), int(pos_offset)

    @staticmethod
    def supported(x: torch.Tensor, dh: int, bias) -> bool:
        return x.is_cuda and x.dtype == torch.bfloat16 and dh in (64, 128) and bias is None


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False, out: torch.Tensor | None = None,
         out_dtype: torch.dtype | None = None, bias: torch.Tensor | None = None,
         residual: torch.Tensor | None = None, accumulate: bool = False, gelu: bool = False,
         alpha: float = 1.0, rope: "RopeEpilogue | None" = None, swiglu_out: torch.Tensor | None = None) -> torch.Tensor:
    """See module docstring. ``a`` is ``[M,K]`` (or ``[K,M]`` when ``a_mn``), ``b`` is ``[N,K]`` (or ``[K,N]``).
    ``rope``: rotate the leading q / k head columns of the output in the epilogue (see ``RopeEpilogue``).
    ``swiglu_out`` [M, N / 2] bf16: ``b`` is [gate rows | up rows]; besides the projection itself the epilogue stores
    silu(gate) * up there (see ``swiglu_epilogue_supported``)."""
    a = _row_major_2d(a)
    b = _row_major_2d(b)
    if a_mn:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    if K != Kb:
        raise ValueError(f"gemm: reduction sizes differ ({K} vs {Kb})")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype or a.dtype, device=a.device)
        if accumulate:
            out.zero_()
    elif out.shape != (M, N):
        out = out.view(M, N)
    native = _use_native(a, b, bias, residual) and out.dtype in (torch.bfloat16, torch.float32) \
        and K % 8 == 0 and out.stride(1) == 1
    if native and (a_mn and M % 8 or b_mn and N % 8 or out.stride(0) % 8):
        native = False
    if native:
        if residual is not None:
            residual = _row_major_2d(residual)
        args = _lib.GemmArgs(
            A=a.data_ptr(), B=b.data_ptr(), C=out.data_ptr(), bias=_lib.p(bias), residual=_lib.p(residual),
            M=M, N=N, K=K, lda=a.stride(0), ldb=b.stride(0), ldc=out.stride(0),
            ldr=residual.stride(0) if residual is not None else 0,
            a_mn_major=int(a_mn), b_mn_major=int(b_mn), c_f32=int(out.dtype == torch.float32),
            accumulate=int(accumulate), act=int(gelu), alpha=float(alpha))
        if swiglu_out is not None:
            args.swiglu_out, args.swiglu_ld = swiglu_out.data_ptr(), swiglu_out.stride(0)
        if rope is not None:
            args.rope_cols, args.rope_dh = rope.cols, rope.dh
            args.rope_inv_freq = rope.inv_freq.data_ptr()
            args.rope_pos = _lib.p(rope.positions) or None
            args.rope_pos_div, args.rope_pos_mod, args.rope_pos_offset = rope.pos_div, 0, rope.pos_offset
        _lib.check(_lib.lib().gv_gemm_bf16(args, _lib.stream_ptr()), "gv_gemm_bf16")
        return out
    if rope is not None or swiglu_out is not None:
        raise _lib.KernelError("gemm: the rotary / gated-activation epilogues need the native kernel (bf16 CUDA operands)")
    if a.is_cuda and a.dtype == torch.bfloat16 and not _lib_fallback_allowed():
        raise _lib.KernelError(f"gemm: shape/stride not supported by the sm_100a kernel: M={M} N={N} K={K}")
    # Reference path (CPU ranks, fp32/fp16 runs): plain PyTorch in the accumulation dtype.
    acc_dtype = torch.float32 if a.dtype in (torch.bfloat16, torch.float16) and not a.is_cuda else a.dtype
    am = (a.t() if a_mn else a).to(acc_dtype)
    bm = (b if b_mn else b.t()).to(acc_dtype)
    c = am @ bm
    if alpha != 1.0:
        c = c * alpha
    if bias is not None:
        c = c + bias.to(acc_dtype)
    if gelu:
        c = torch.nn.functional.gelu(c, approximate="tanh")
    if residual is not None:
        c = c + residual.reshape(M, N).to(acc_dtype)
    if accumulate:
        out.add_(c.to(out.dtype))
    else:
        out.copy_(c)
    return out


def swiglu_epilogue_supported(x: torch.Tensor, w_up: torch.Tensor) -> bool:
    """The gated-activation epilogue wants bf16 CUDA operands in natural storage and an FFN width that is a multiple of
    128 (one output tile = 128 gate columns + the 128 up columns of the same hidden units)."""
    return (_use_native(x, w_up) and w_up.dim() == 2 and w_up.shape[0] % 256 == 0 and w_up.shape[1] % 8 == 0
            and w_up.stride(1) == 1 and w_up.stride(0) % 8 == 0 and w_up.data_ptr() % 16 == 0)


def head_xent_supported(x: torch.Tensor, W: torch.Tensor) -> bool:
    """The cross-entropy epilogues need bf16 CUDA operands in their natural (K-major) storage."""
    return (_use_native(x, W) and x.dim() == 2 and W.dim() == 2 and x.shape[1] == W.shape[1] and x.shape[1] % 8 == 0
            and W.shape[0] % 8 == 0          # the backward twin stores a [tokens, vocab shard] bf16 gradient (row stride % 8)
            and x.stride(1) == 1 and W.stride(1) == 1 and x.stride(0) % 8 == 0 and W.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and W.data_ptr() % 16 == 0)


def _head_args(x, W, C):
    M, K = x.shape
    N = W.shape[0]
    return _lib.GemmArgs(A=x.data_ptr(), B=W.data_ptr(), C=_lib.p(C), bias=0, residual=0, M=M, N=N, K=K, lda=x.stride(0),
                         ldb=W.stride(0), ldc=N if C is None else C.stride(0), ldr=0, a_mn_major=0, b_mn_major=0, c_f32=0,
                         accumulate=0, act=0, alpha=1.0)


def head_xent_stats(x: torch.Tensor, W: torch.Tensor, labels: torch.Tensor, vocab_start: int = 0, ignore_index: int = -100):
    """Language-model head forward without logits: per row (max, sum exp(logit - max), target logit or 0) over this
    rank's vocabulary shard ``W`` [V_local, K], computed in the epilogue of the head GEMM from its fp32 accumulators."""
    M, N = x.shape[0], W.shape[0]
    tiles = (N + 255) // 256
    stats = torch.empty(M, tiles, 2, dtype=torch.float32, device=x.device)
    target = torch.zeros(M, dtype=torch.float32, device=x.device)
    labels = labels.reshape(-1).to(torch.int64).contiguous()
    xa = _lib.XentArgs(mode=1, labels=labels.data_ptr(), vocab_start=int(vocab_start), ignore_index=int(ignore_index),
                       stats=stats.data_ptr(), target=target.data_ptr(), lse=0, gscale=0)
    _lib.check(_lib.lib().gv_gemm_xent(_head_args(x, W, None), xa, _lib.stream_ptr()), "gv_gemm_xent(stats)")
    mx = stats[:, :, 0].max(dim=1).values
    se = (stats[:, :, 1] * torch.exp(stats[:, :, 0] - mx.unsqueeze(1))).sum(dim=1)
    return mx, se, target


def head_xent_grad(x: torch.Tensor, W: torch.Tensor, labels: torch.Tensor, lse: torch.Tensor, gscale: torch.Tensor,
                   vocab_start: int = 0, ignore_index: int = -100) -> torch.Tensor:
    """d loss / d logits (bf16 [M, V_local]) from recomputed logits: (softmax - onehot) * gscale[row], written by the
    epilogue of the head GEMM; ``lse`` is the log-sum-exp over the whole vocabulary."""
    M, N = x.shape[0], W.shape[0]
    out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    labels = labels.reshape(-1).to(torch.int64).contiguous()
    lse = lse.float().contiguous()
    gscale = gscale.float().contiguous()
    xa = _lib.XentArgs(mode=2, labels=labels.data_ptr(), vocab_start=int(vocab_start), ignore_index=int(ignore_index),
                       stats=0, target=0, lse=lse.data_ptr(), gscale=gscale.data_ptr())
    _lib.check(_lib.lib().gv_gemm_xent(_head_args(x, W, out), xa, _lib.stream_ptr()), "gv_gemm_xent(grad)")
    return out


def _lib_fallback_allowed() -> bool:
    # Odd shapes (K or leading dimensions not multiples of 8) only occur in tiny unit-test models;
    # they take the PyTorch path instead of failing.
    return True
