"""Micro-benchmarks of the native kernels against library baselines, with roofline fractions.

    python -m hetu_galvatron_b200.ops.kernel_bench --op gemm            # Llama-7B GEMM shapes, fwd / dgrad / wgrad
    python -m hetu_galvatron_b200.ops.kernel_bench --op attention       # causal flash attention fwd / bwd
    python -m hetu_galvatron_b200.ops.kernel_bench --op elementwise     # norm / swiglu / rope / cross-entropy / adamw
    python -m hetu_galvatron_b200.ops.kernel_bench --op window_attention  # Swin windows: additive bias + shift mask
    python -m hetu_galvatron_b200.ops.kernel_bench --op mma_issue       # cycles per tcgen05.mma by tile shape
    python -m hetu_galvatron_b200.ops.kernel_bench --op gemm --m 8192 --n 4096 --k 4096 --iters 2 --no-baseline

Timing: CUDA events on the launching stream, 3 warm-up calls, a 256 MiB write between timed calls to flush L2, median
of ``--iters`` calls. Fractions are "of measured": the denominators are the copy bandwidth and cuBLAS bf16 throughput
in ``MEASURED_PEAKS.json`` at the repository root (fallback 6.65 TB/s and 1.59 PFLOP/s when that file is absent).
The single-shape form with ``--no-baseline`` is the small case profiler captures are taken on.
"""
from __future__ import annotations

import argparse
import json
import math
import os

import torch

from . import _lib
from . import functional as Fn
from .gemm import gemm


def peaks() -> dict:
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        d = json.load(open(os.path.join(here, "MEASURED_PEAKS.json")))
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


_FLUSH = None


def timeit(fn, iters: int = 10, flush: bool = True) -> float:
    global _FLUSH
    if flush and _FLUSH is None:
        _FLUSH = torch.empty(256 * 2 ** 20, dtype=torch.uint8, device="cuda")
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush:
            _FLUSH.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def bench_gemm(shapes, iters: int, baseline: bool, modes=("fwd", "dgrad", "wgrad")):
    pk = peaks()
    out = []
    for (M, N, K) in shapes:
        for mode in modes:
            x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
            w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
            dy = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
            if mode == "fwd":
                ours, lib = (lambda: gemm(x, w)), (lambda: x @ w.t())
            elif mode == "dgrad":
                ours, lib = (lambda: gemm(dy, w, b_mn=True)), (lambda: dy @ w)
            else:
                ours, lib = (lambda: gemm(dy, x, a_mn=True, b_mn=True)), (lambda: dy.t() @ x)
            t = timeit(ours, iters)
            fl = 2.0 * M * N * K
            r = {"op": "gemm", "mode": mode, "M": M, "N": N, "K": K, "ms": round(t, 4), "tflops": round(fl / t / 1e9, 1),
                 "frac_of_%s_cublas_peak" % pk["source"]: round(fl / t / 1e9 / pk["bf16_tflops"], 3)}
            if baseline:
                tl = timeit(lib, iters)
                r.update(cublas_ms=round(tl, 4), cublas_tflops=round(fl / tl / 1e9, 1), vs_cublas=round(tl / t, 3))
            print(json.dumps(r), flush=True)
            out.append(r)
            del x, w, dy
    return out


def bench_attention(cases, iters: int, baseline: bool):
    import torch.nn.functional as F
    pk = peaks()
    out = []
    for (b, s, h, hk, dh) in cases:
        qkv = torch.randn(b, s, (h + 2 * hk) * dh, device="cuda", dtype=torch.bfloat16)
        q = qkv[..., :h * dh].view(b, s, h, dh)
        k = qkv[..., h * dh:(h + hk) * dh].view(b, s, hk, dh)
        v = qkv[..., (h + hk) * dh:].view(b, s, hk, dh)
        sc = 1.0 / math.sqrt(dh)
        o, lse = Fn.attention_fwd(q, k, v, True, sc)
        do = torch.randn_like(o)
        tf = timeit(lambda: Fn.attention_fwd(q, k, v, True, sc), iters)
        tb = timeit(lambda: Fn.attention_bwd(do, q, k, v, o, lse, True, sc), iters)
        fl = 4.0 * b * h * s * s * dh / 2
        r = {"op": "attention", "b": b, "s": s, "hq": h, "hk": hk, "dh": dh, "fwd_ms": round(tf, 4),
             "fwd_tflops": round(fl / tf / 1e9, 1), "bwd_ms": round(tb, 4), "bwd_tflops": round(2.5 * fl / tb / 1e9, 1),
             "fwd_frac_of_%s_cublas_peak" % pk["source"]: round(fl / tf / 1e9 / pk["bf16_tflops"], 3),
             "bwd_frac_of_%s_cublas_peak" % pk["source"]: round(2.5 * fl / tb / 1e9 / pk["bf16_tflops"], 3)}
        if baseline and h == hk:
            qq, kk, vv = (t.transpose(1, 2) for t in (q, k, v))
            tl = timeit(lambda: F.scaled_dot_product_attention(qq, kk, vv, is_causal=True), iters)
            r.update(sdpa_fwd_ms=round(tl, 4), sdpa_fwd_tflops=round(fl / tl / 1e9, 1))
        print(json.dumps(r), flush=True)
        out.append(r)
    return out


# (images, resolution in tokens, window side, heads, head size): the four stages of Swin-L / 384 and stage 1 of Swin-H / 224
WINDOW_CASES = [(8, 96, 12, 6, 32), (8, 48, 12, 12, 32), (8, 24, 12, 24, 32), (8, 12, 12, 48, 32), (32, 56, 7, 11, 32)]


def bench_window_attention(cases, iters: int, baseline: bool):
    """Windowed attention with relative-position bias and shifted-window regions (group ids): windows are batch elements of
    the attention kernels. Baseline: torch's scaled_dot_product_attention given the materialised [windows, heads, s, s]
    additive mask (bias + -30000 between regions)."""
    import torch.nn.functional as F
    from . import autograd as A

    out = []
    for (imgs, res, ws, h, dh) in cases:
        nw = (res // ws) ** 2
        bw, s = imgs * nw, ws * ws
        q, k, v = (torch.randn(bw, s, h, dh, device="cuda", dtype=torch.bfloat16, requires_grad=True) for _ in range(3))
        bias = torch.randn(h, s, s, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        ids = torch.randint(0, 3, (nw, s), device="cuda", dtype=torch.int32)          # regions glued together by a shift
        mask = torch.zeros(nw, s, s, device="cuda", dtype=torch.bfloat16).masked_fill(ids[:, :, None] != ids[:, None, :], -30000.0)
        sc = 1.0 / math.sqrt(dh)
        o = A.biased_attention(q, k, v, bias, None, ids, sc)
        do = torch.randn_like(o)
        tf = timeit(lambda: A.biased_attention(q, k, v, bias, None, ids, sc), iters)
        tfb = timeit(lambda: torch.autograd.grad(A.biased_attention(q, k, v, bias, None, ids, sc), [q, k, v, bias], do), iters)
        fl = 4.0 * bw * h * s * s * dh
        nbytes = 4 * bw * s * h * dh * 2          # q, k, v read, o written
        r = {"op": "window_attention", "images": imgs, "tokens": res * res, "window": ws, "heads": h, "dh": dh, "windows": bw,
             "fwd_ms": round(tf, 4), "fwd_tflops": round(fl / tf / 1e9, 1), "fwd_gbs": round(nbytes / tf / 1e6, 1),
             "fwd_bwd_ms": round(tfb, 4), "fwd_bwd_tflops": round(3.5 * fl / tfb / 1e9, 1)}
        if baseline:
            qq, kk, vv = (t.detach().transpose(1, 2).requires_grad_(True) for t in (q, k, v))
            bb = bias.detach().requires_grad_(True)

            def sdpa():
                m = (bb.unsqueeze(0).unsqueeze(0) + mask.view(1, nw, 1, s, s)).expand(imgs, -1, -1, -1, -1).reshape(bw, h, s, s)
                return F.scaled_dot_product_attention(qq, kk, vv, attn_mask=m)

            dd = do.transpose(1, 2)
            tl = timeit(sdpa, iters)
            tlb = timeit(lambda: torch.autograd.grad(sdpa(), [qq, kk, vv, bb], dd), iters)
            r.update(sdpa_fwd_ms=round(tl, 4), sdpa_fwd_bwd_ms=round(tlb, 4), fwd_speedup=round(tl / tf, 2),
                     fwd_bwd_speedup=round(tlb / tfb, 2))
        print(json.dumps(r), flush=True)
        out.append(r)
    return out


def bench_window_breakdown(iters: int, case=(8, 96, 12, 6, 32)):
    """Kernel-only times of one windowed-attention case (``ops.attention.fwd / bwd`` called directly): what the bias, the
    group ids, the general additive mask and the bias gradient each add to the plain kernels."""
    from . import attention as at

    imgs, res, ws, h, dh = case
    nw = (res // ws) ** 2
    bw, s = imgs * nw, ws * ws
    q, k, v = (torch.randn(bw, s, h, dh, device="cuda", dtype=torch.bfloat16) for _ in range(3))
    bias = torch.randn(h, s, s, device="cuda")
    ids = torch.randint(0, 3, (nw, s), device="cuda", dtype=torch.int32)
    mask = torch.zeros(nw, s, s, device="cuda").masked_fill(ids[:, :, None] != ids[:, None, :], -30000.0)
    a_bias, a_ids, a_mask = at.Additive(s, s, bias), at.Additive(s, s, bias, None, ids), at.Additive(s, s, bias, mask, None)
    sc = 1.0 / math.sqrt(dh)
    o, lse = at.fwd(q, k, v, False, sc, additive=a_ids)
    do = torch.randn_like(o)
    dbias = torch.zeros(a_ids.bias.shape, dtype=torch.float32, device="cuda")
    r = {"op": "window_attention_breakdown", "images": imgs, "tokens": res * res, "window": ws, "heads": h, "dh": dh, "windows": bw}
    r["fwd_plain_ms"] = timeit(lambda: at.fwd(q, k, v, False, sc), iters)
    r["fwd_bias_ms"] = timeit(lambda: at.fwd(q, k, v, False, sc, additive=a_bias), iters)
    r["fwd_bias_ids_ms"] = timeit(lambda: at.fwd(q, k, v, False, sc, additive=a_ids), iters)
    r["fwd_bias_mask_ms"] = timeit(lambda: at.fwd(q, k, v, False, sc, additive=a_mask), iters)
    r["bwd_plain_ms"] = timeit(lambda: at.bwd(do, q, k, v, o, lse, False, sc), iters)
    r["bwd_bias_ms"] = timeit(lambda: at.bwd(do, q, k, v, o, lse, False, sc, additive=a_bias), iters)
    r["bwd_bias_ids_ms"] = timeit(lambda: at.bwd(do, q, k, v, o, lse, False, sc, additive=a_ids), iters)
    r["bwd_bias_ids_dbias_ms"] = timeit(lambda: at.bwd(do, q, k, v, o, lse, False, sc, additive=a_ids, dbias=dbias), iters)
    r["bwd_bias_mask_dbias_ms"] = timeit(lambda: at.bwd(do, q, k, v, o, lse, False, sc, additive=a_mask, dbias=dbias), iters)
    r["additive_build_ms"] = timeit(lambda: at.Additive(s, s, bias, None, ids), iters)
    r = {k2: (round(v2, 4) if isinstance(v2, float) else v2) for k2, v2 in r.items()}
    print(json.dumps(r), flush=True)
    return [r]


def bench_elementwise(tokens: int, hidden: int, ffn: int, vocab: int, iters: int):
    pk = peaks()
    dev, bf = "cuda", torch.bfloat16
    out = []

    def rec(name, nbytes, fn):
        t = timeit(fn, iters)
        r = {"op": name, "ms": round(t, 4), "GBps": round(nbytes / t / 1e6, 1),
             "frac_of_%s_copy_bw" % pk["source"]: round(nbytes / t / 1e6 / pk["hbm_gbs"], 3)}
        print(json.dumps(r), flush=True)
        out.append(r)

    x = torch.randn(tokens, hidden, device=dev, dtype=bf)
    w = torch.ones(hidden, device=dev, dtype=bf)
    rec("rmsnorm_fwd", 2 * x.numel() * 2, lambda: Fn.rmsnorm_fwd(x, w, 1e-5))
    y, _, rstd = Fn.rmsnorm_fwd(x, w, 1e-5)
    dw = torch.zeros(hidden, device=dev, dtype=torch.float32)
    rec("rmsnorm_bwd", 3 * x.numel() * 2, lambda: Fn.rmsnorm_bwd(y, x, w, rstd, None, dw))
    gu = torch.randn(tokens, 2 * ffn, device=dev, dtype=bf)
    rec("swiglu_fwd", 3 * tokens * ffn * 2, lambda: Fn.swiglu_fwd(gu))
    da = torch.randn(tokens, ffn, device=dev, dtype=bf)
    rec("swiglu_bwd", 5 * tokens * ffn * 2, lambda: Fn.swiglu_bwd(da, gu))
    n = 200 * 2 ** 20
    master = torch.randn(n, device=dev)
    m, v = torch.zeros_like(master), torch.zeros_like(master)
    g = torch.randn(n, device=dev, dtype=bf)
    low = torch.empty(n, device=dev, dtype=bf)
    rec("adamw_step", n * (3 * 4 * 2 + 2 + 2), lambda: Fn.adamw_step_(master, m, v, g, low, lr=1e-4, beta1=0.9, beta2=0.95,
                                                                     eps=1e-8, weight_decay=0.1, step=3, grad_scale=1.0,
                                                                     clip_coef=None))
    return out


def bench_mma_issue(reps: int = 2000):
    """Cycles per ``tcgen05.mma`` (bf16, K = 16) issued back to back by one thread, per instruction shape."""
    import ctypes

    lib = _lib.lib()
    buf = torch.zeros(4, dtype=torch.int64, device="cuda")
    out = []
    forms = [(0, 128, 256), (0, 128, 128), (0, 128, 64), (0, 128, 32), (0, 64, 256), (0, 64, 128),
             (1, 256, 256), (1, 256, 128), (1, 128, 256)]
    for pair, m, n in forms:
        for r in (10, reps):           # first a short warm-up launch
            _lib.check(lib.gv_bench_mma_issue(pair, m, n, r, ctypes.c_void_p(buf.data_ptr()),
                                              ctypes.c_void_p(_lib.stream_ptr())), "gv_bench_mma_issue")
            torch.cuda.synchronize()
        total, issue, ok = (int(v) for v in buf[:3].tolist())
        ideal = m * n * 16 * 2 / 8192.0 / (2 if pair else 1)      # 8192 dense bf16 FLOP per clock per SM
        rec = {"op": "mma_issue", "form": "cta_group::2" if pair else "cta_group::1", "M": m, "N": n,
               "cycles_per_mma": round(total / (4.0 * reps), 1), "ideal_cycles": ideal, "completed": bool(ok)}
        print(json.dumps(rec), flush=True)
        out.append(rec)
    return out


LLAMA7B_GEMMS = [(8192, 12288, 4096), (8192, 4096, 4096), (8192, 22016, 4096), (8192, 4096, 11008), (8192, 32000, 4096)]
ATTN_CASES = [(2, 4096, 32, 32, 128), (1, 8192, 32, 32, 128), (4, 4096, 16, 16, 128), (2, 4096, 32, 8, 128)]


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="gemm", choices=["gemm", "attention", "window_attention", "elementwise", "mma_issue", "all"])
    ap.add_argument("--m", type=int, default=0)
    ap.add_argument("--n", type=int, default=0)
    ap.add_argument("--k", type=int, default=0)
    ap.add_argument("--mode", default=None, choices=[None, "fwd", "dgrad", "wgrad"])
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--seq", type=int, default=0)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=0)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--no-baseline", action="store_true")
    ap.add_argument("--breakdown", action="store_true", help="window_attention: kernel-only times of the optional score terms")
    ap.add_argument("--out", default=None)
    a = ap.parse_args(argv)
    torch.cuda.set_device(0)
    res = []
    if a.op in ("gemm", "all"):
        shapes = [(a.m, a.n, a.k)] if a.m else LLAMA7B_GEMMS
        res += bench_gemm(shapes, a.iters, not a.no_baseline, modes=(a.mode,) if a.mode else ("fwd", "dgrad", "wgrad"))
    if a.op in ("attention", "all"):
        cases = [(a.batch, a.seq, a.heads, a.kv_heads or a.heads, 128)] if a.seq else ATTN_CASES
        res += bench_attention(cases, a.iters, not a.no_baseline)
    if a.op in ("window_attention", "all"):
        res += bench_window_breakdown(a.iters) if a.breakdown else bench_window_attention(WINDOW_CASES, a.iters, not a.no_baseline)
    if a.op in ("elementwise", "all"):
        res += bench_elementwise(8192, 4096, 11008, 32000, a.iters)
    if a.op == "mma_issue":
        res += bench_mma_issue()
    err = _lib.read_error()
    print(json.dumps({"kernel_error": err, "peaks": peaks()}), flush=True)
    if a.out:
        json.dump(res, open(a.out, "w"), indent=1)


if __name__ == "__main__":
    main()
