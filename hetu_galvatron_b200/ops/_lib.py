"""ctypes loader for the sm_100a kernel library (``_lib/libgvkernels.so``).

The library has a plain C ABI (csrc/include/gv_kernels.h): raw device pointers plus a stream.
On a machine with a GPU a missing library is an error -- there is no silent fallback to
PyTorch kernels for bf16 CUDA tensors.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_float, c_int, c_longlong, c_uint, c_ulonglong, c_void_p

import torch

from .. import _build

_LIB = None

# Kernel launches per library call (for launch accounting in benchmarks).
KERNELS_PER_CALL = {"gv_attn_bwd": 3, "gv_read_error": 0, "gv_norm_bwd_scratch_elems": 0, "gv_rmsnorm_bwd": 2,
                    "gv_layernorm_bwd": 2, "gv_device_sm_count": 0}
LAUNCH_COUNT = 0


class _CountingLib:
    """Proxy over the CDLL that counts kernel launches made through the library."""

    def __init__(self, cdll):
        object.__setattr__(self, "_cdll", cdll)
        object.__setattr__(self, "_cache", {})

    def __getattr__(self, name):
        cache = object.__getattribute__(self, "_cache")
        fn = cache.get(name)
        if fn is None:
            raw = getattr(object.__getattribute__(self, "_cdll"), name)
            if not name.startswith("gv_") or not callable(raw):
                return raw
            n = KERNELS_PER_CALL.get(name, 1)

            def fn(*args, _raw=raw, _n=n):
                global LAUNCH_COUNT
                LAUNCH_COUNT += _n
                return _raw(*args)

            fn.raw = raw
            cache[name] = fn
        return fn

    def __setattr__(self, name, value):
        setattr(object.__getattribute__(self, "_cdll"), name, value)


class GemmArgs(Structure):
    _fields_ = [
        ("A", c_void_p), ("B", c_void_p), ("C", c_void_p), ("bias", c_void_p), ("residual", c_void_p),
        ("M", c_int), ("N", c_int), ("K", c_int),
        ("lda", c_int), ("ldb", c_int), ("ldc", c_int), ("ldr", c_int),
        ("a_mn_major", c_int), ("b_mn_major", c_int),
        ("c_f32", c_int), ("accumulate", c_int), ("act", c_int),
        ("alpha", c_float),
        ("rope_cols", c_int), ("rope_dh", c_int), ("rope_inv_freq", c_void_p), ("rope_pos", c_void_p),
        ("rope_pos_div", c_int), ("rope_pos_mod", c_int), ("rope_pos_offset", c_int),
        ("swiglu_out", c_void_p), ("swiglu_ld", c_int),
    ]


class XentArgs(Structure):
    _fields_ = [("mode", c_int), ("labels", c_void_p), ("vocab_start", c_longlong), ("ignore_index", c_longlong),
                ("stats", c_void_p), ("target", c_void_p), ("lse", c_void_p), ("gscale", c_void_p)]


class AttnArgs(Structure):
    _fields_ = [
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("o", c_void_p), ("lse", c_void_p),
        ("dout", c_void_p), ("dq", c_void_p), ("dk", c_void_p), ("dv", c_void_p),
        ("dq_accum", c_void_p), ("delta", c_void_p),
        ("b", c_int), ("sq", c_int), ("sk", c_int), ("hq", c_int), ("hk", c_int), ("dh", c_int),
        ("q_stride_b", c_longlong), ("q_stride_s", c_longlong), ("q_stride_h", c_longlong),
        ("k_stride_b", c_longlong), ("k_stride_s", c_longlong), ("k_stride_h", c_longlong),
        ("v_stride_b", c_longlong), ("v_stride_s", c_longlong), ("v_stride_h", c_longlong),
        ("o_stride_b", c_longlong), ("o_stride_s", c_longlong), ("o_stride_h", c_longlong),
        ("do_stride_b", c_longlong), ("do_stride_s", c_longlong), ("do_stride_h", c_longlong),
        ("dq_stride_b", c_longlong), ("dq_stride_s", c_longlong), ("dq_stride_h", c_longlong),
        ("dk_stride_b", c_longlong), ("dk_stride_s", c_longlong), ("dk_stride_h", c_longlong),
        ("dv_stride_b", c_longlong), ("dv_stride_s", c_longlong), ("dv_stride_h", c_longlong),
        ("causal", c_int), ("scale", c_float), ("kv_lens", c_void_p),
        ("dq_rope_inv_freq", c_void_p), ("dq_rope_pos", c_void_p), ("dq_rope_pos_offset", c_int),
        ("dropout_p", c_float), ("dropout_seed", c_ulonglong), ("dropout_head_offset", c_int),
        ("bias", c_void_p), ("bias_t", c_void_p), ("mask", c_void_p), ("ids", c_void_p), ("mask_n", c_int), ("bias_ld", c_int),
        ("dbias", c_void_p),
    ]


def available() -> bool:
    """True when the kernel library can be used (a CUDA device is present)."""
    return torch.cuda.is_available()


def lib():
    global _LIB
    if _LIB is None:
        path = _build.cuda_lib_path()
        if not path.exists():
            path = _build.build_cuda()
        cdll = ctypes.CDLL(str(path))
        cdll.gv_read_error.argtypes = [POINTER(c_uint)]
        cdll.gv_read_error.restype = c_int
        cdll.gv_gemm_bf16.argtypes = [POINTER(GemmArgs), c_void_p]
        cdll.gv_gemm_bf16.restype = c_int
        cdll.gv_gemm_xent.argtypes = [POINTER(GemmArgs), POINTER(XentArgs), c_void_p]
        cdll.gv_gemm_xent.restype = c_int
        _LIB = _CountingLib(cdll)
    return _LIB


def launch_count() -> int:
    return LAUNCH_COUNT


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


class KernelError(RuntimeError):
    pass


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise KernelError(f"{what} failed to launch (code {rc})")


def read_error():
    """Return the first error record written by a bounded device wait, or None."""
    buf = (c_uint * 4)()
    rc = lib().gv_read_error(buf)
    if rc == 0:
        return None
    return {"code": buf[0], "site": buf[0] >> 16, "block": buf[1], "aux0": buf[2], "aux1": buf[3]}


def p(t) -> int:
    return 0 if t is None else t.data_ptr()
