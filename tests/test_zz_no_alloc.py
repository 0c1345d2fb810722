"""The allocation-free attention backward (csrc/no_alloc.cu), called through its exported C symbol.

Some programs that embed this library own all device memory themselves (a pool that was sized to whatever was
free) and forbid cudaMalloc on their hot path; for them the library ships one entry point whose scratch memory is
a fixed device array inside the library. This test calls it with ctypes exactly as such a C caller would, twice
in a row (the scratch is shared and keeps the previous call's contents), and checks the gradients against the
regular entry point. The file name sorts last so a run that stops at the first failure has already run the
other tests."""
import ctypes
import math

import pytest
import torch

from hetu_galvatron_b200 import _build
from hetu_galvatron_b200.ops import _lib
from hetu_galvatron_b200.ops import functional as Fn

pytestmark = pytest.mark.gpu


def _args(q, k, v, o, lse, dout, dq, dk, dv, causal, scale):
    b, sq, hq, dh = q.shape
    a = _lib.AttnArgs(q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), o=o.data_ptr(), lse=lse.data_ptr(),
                      dout=dout.data_ptr(), dq=dq.data_ptr(), dk=dk.data_ptr(), dv=dv.data_ptr(), dq_accum=None, delta=None,
                      b=b, sq=sq, sk=k.shape[1], hq=hq, hk=k.shape[2], dh=dh, causal=int(causal), scale=float(scale))
    for name, t in (("q", q), ("k", k), ("v", v), ("o", o), ("do", dout), ("dq", dq), ("dk", dk), ("dv", dv)):
        setattr(a, name + "_stride_b", t.stride(0))
        setattr(a, name + "_stride_s", t.stride(1))
        setattr(a, name + "_stride_h", t.stride(2))
    return a


def test_no_alloc_attention_backward_matches_regular_entry_point():
    cdll = ctypes.CDLL(str(_build.cuda_lib_path()))
    fn = cdll.gv_attn_bwd_noalloc
    fn.argtypes = [ctypes.POINTER(_lib.AttnArgs), ctypes.c_void_p]
    fn.restype = ctypes.c_int
    strerror = cdll.gv_attn_bwd_noalloc_strerror
    strerror.argtypes = [ctypes.c_int]
    strerror.restype = ctypes.c_char_p
    torch.manual_seed(0)
    stream = torch.cuda.current_stream().cuda_stream
    for call, (b, s, hq, hk, dh, causal) in enumerate([(2, 384, 4, 2, 128, True), (1, 200, 2, 2, 64, False)]):
        q = torch.randn(b, s, hq, dh, device="cuda", dtype=torch.bfloat16)
        k = torch.randn(b, s, hk, dh, device="cuda", dtype=torch.bfloat16)
        v = torch.randn(b, s, hk, dh, device="cuda", dtype=torch.bfloat16)
        scale = 1.0 / math.sqrt(dh)
        o, lse = Fn.attention_fwd(q, k, v, causal, scale)
        dout = torch.randn_like(o)
        ref = Fn.attention_bwd(dout, q, k, v, o, lse, causal, scale)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        a = _args(q, k, v, o, lse, dout, dq, dk, dv, causal, scale)
        if call == 0:
            # warm-up: the first call on a device resolves the scratch address and sets the kernels' shared-memory
            # limit once; free memory is compared only around calls made after that
            assert fn(a, stream) == 0
            torch.cuda.synchronize()
        # the driver's own count of free device memory sees any cudaMalloc, whoever made it (the caching
        # allocator's statistics would only see PyTorch's)
        free_before = torch.cuda.mem_get_info()[0]
        rc = fn(a, stream)
        assert rc == 0, strerror(rc)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before
        for got, want in zip((dq, dk, dv), ref):
            err = (got.float() - want.float()).abs().max() / (want.float().abs().max() + 1e-6)
            assert err.item() < 3e-2, (call, err.item())
    # beyond the fixed scratch: refused with a clear message, nothing launched
    big = _lib.AttnArgs(b=8, sq=8192, sk=8192, hq=32, hk=32, dh=128)
    free_before = torch.cuda.mem_get_info()[0]
    rc = fn(big, stream)
    assert rc == -2401 and b"too large" in strerror(rc)
    # a missing or inconsistent argument block has its own code (and must not divide by a zero head count)
    assert fn(None, stream) == -2404 and b"bad arguments" in strerror(-2404)
    assert fn(_lib.AttnArgs(b=1, sq=128, sk=128, hq=0, hk=0, dh=128), stream) == -2404
    assert torch.cuda.mem_get_info()[0] == free_before
    assert _lib.read_error() is None
