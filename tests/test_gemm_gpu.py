"""tcgen05 GEMM vs a PyTorch fp32 reference (all operand majors, epilogues, ragged sizes)."""
import pytest
import torch

from hetu_galvatron_b200.ops import gemm
from hetu_galvatron_b200.ops import _lib

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    af = (a.t() if a_mn else a).float()
    bf = (b if b_mn else b.t()).float()
    return af @ bf


def _check(c, ref, K):
    err = (c.float() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    assert err / scale < 2e-2, f"rel err {err / scale}"
    assert _lib.read_error() is None


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (384, 768, 1024), (1000, 520, 136), (4096, 4096, 4096),
                                   (72, 40, 8), (136, 264, 72)])
def test_gemm_majors(a_mn, b_mn, M, N, K):
    torch.manual_seed(0)
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda", dtype=torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda", dtype=torch.bfloat16)
    c = gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    torch.cuda.synchronize()
    _check(c, _ref(a, b, a_mn, b_mn), K)


def test_gemm_is_bitwise_repeatable():
    """Fixed tile schedule and fixed accumulation order: the same inputs give the same bits, single-CTA and pair tiles."""
    torch.manual_seed(1)
    for M, N, K in ((1000, 520, 136), (8192, 4096, 1024)):
        a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
        first = gemm(a, b).clone()
        for _ in range(3):
            assert torch.equal(gemm(a, b), first)
    assert _lib.read_error() is None


def test_gemm_epilogues():
    torch.manual_seed(1)
    M, N, K = 512, 1024, 512
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    ref = a.float() @ b.float().t()
    _check(gemm(a, b, bias=bias), ref + bias.float(), K)
    _check(gemm(a, b, residual=res), ref + res.float(), K)
    _check(gemm(a, b, bias=bias, gelu=True), torch.nn.functional.gelu(ref + bias.float(), approximate="tanh"), K)
    acc = torch.randn(M, N, device="cuda", dtype=torch.float32)
    acc0 = acc.clone()
    gemm(a, b, out=acc, accumulate=True)
    _check(acc, acc0 + ref, K)
    out32 = gemm(a, b, out_dtype=torch.float32)
    _check(out32, ref, K)
    accb = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    accb0 = accb.clone()
    gemm(a, b, out=accb, accumulate=True)
    _check(accb, accb0.float() + ref, K)


def test_gemm_linear_grads_match_torch():
    torch.manual_seed(2)
    M, N, K = 1024, 768, 512
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.05
    dy = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    dx = gemm(dy, w, b_mn=True)
    dw = gemm(dy, x, a_mn=True, b_mn=True, out_dtype=torch.float32)
    _check(dx, dy.float() @ w.float(), N)
    _check(dw, dy.float().t() @ x.float(), M)


def test_gemm_strided_views():
    torch.manual_seed(3)
    big = torch.randn(512, 1024, device="cuda", dtype=torch.bfloat16)
    a = big[:, 256:768]  # row stride 1024, 16-byte aligned offset
    b = torch.randn(384, 512, device="cuda", dtype=torch.bfloat16)
    _check(gemm(a, b), a.float() @ b.float().t(), 512)


PAIR_SCRIPT = r"""
import json, sys, torch
sys.path.insert(0, %r)
from hetu_galvatron_b200.ops.gemm import gemm
from hetu_galvatron_b200.ops import _lib
torch.manual_seed(0)
out = {}
for (M, N, K) in [(256, 256, 64), (512, 768, 128), (1000, 1032, 200), (4096, 2048, 512), (300, 256, 4096)]:
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    res = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    ref = a.float() @ w.float().t()
    y = gemm(a, w).float()
    out["%%d_%%d_%%d" %% (M, N, K)] = ((y - ref).abs().max() / ref.abs().max()).item()
    y2 = gemm(a, w, bias=bias, residual=res).float()
    ref2 = ref + bias.float() + res.float()
    out["%%d_%%d_%%d_epi" %% (M, N, K)] = ((y2 - ref2).abs().max() / ref2.abs().max()).item()
    acc = torch.randn(M, N, device="cuda", dtype=torch.float32)
    ref3 = acc + ref
    gemm(a, w, out=acc, accumulate=True)
    out["%%d_%%d_%%d_acc" %% (M, N, K)] = ((acc - ref3).abs().max() / ref3.abs().max()).item()
    dy = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
    ref4 = dy.float() @ w.float()                       # input gradient: B used as stored [N, K] = MN-major
    out["%%d_%%d_%%d_dgrad" %% (M, N, K)] = ((gemm(dy, w, b_mn=True).float() - ref4).abs().max() / ref4.abs().max()).item()
    ref5 = dy.float().t() @ a.float()                   # weight gradient: both operands MN-major, reduction over M
    dw = torch.zeros(N, K, device="cuda", dtype=torch.float32)
    gemm(dy, a, a_mn=True, b_mn=True, out=dw, accumulate=True)
    out["%%d_%%d_%%d_wgrad" %% (M, N, K)] = ((dw - ref5).abs().max() / ref5.abs().max()).item()
torch.cuda.synchronize()
out["error"] = _lib.read_error()
print("PAIR " + json.dumps(out))
"""


@pytest.mark.gpu
def test_pair_kernel_matches_fp32_reference():
    """The two-CTA (cta_group::2) kernel, forced on for every K-major shape, against fp32 matmul; bias + residual and
    fp32-accumulate epilogues; M and N tails inside a 256 x 256 pair tile."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, GV_GEMM_PAIR="2")
    r = subprocess.run([sys.executable, "-c", PAIR_SCRIPT % root], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("PAIR ")][0]
    res = json.loads(line[5:])
    assert res.pop("error") is None
    for k, v in res.items():
        assert v < 1e-2, (k, v, res)


@pytest.mark.parametrize("M,V,K,vocab_start", [(256, 1000, 256, 0), (300, 4096, 512, 4096), (8192, 32000, 1024, 0), (128, 264, 64, 0)])
def test_lm_head_cross_entropy_epilogues(M, V, K, vocab_start):
    """Head GEMM whose epilogue computes the cross-entropy statistics (no logits stored), and its backward twin whose
    epilogue writes (softmax - onehot) * dloss, against fp32 PyTorch."""
    from hetu_galvatron_b200.ops.gemm import head_xent_grad, head_xent_stats, head_xent_supported
    torch.manual_seed(0)
    x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    W = (torch.randn(V, K, device="cuda") * 0.2).bfloat16()
    labels = torch.randint(vocab_start - 50 if vocab_start else 0, vocab_start + V + (50 if vocab_start else 0), (M,), device="cuda")
    labels[::7] = -100
    assert head_xent_supported(x, W)
    mx, se, tg = head_xent_stats(x, W, labels, vocab_start)
    logits = x.float() @ W.float().t()
    mr = logits.max(-1).values
    sr = (logits - mr.unsqueeze(-1)).exp().sum(-1)
    local = labels - vocab_start
    inside = (labels != -100) & (local >= 0) & (local < V)
    tr = torch.where(inside, logits.gather(1, local.clamp(0, V - 1).unsqueeze(1)).squeeze(1), torch.zeros_like(mr))
    assert (mx - mr).abs().max().item() < 1e-3
    assert ((se.log() + mx) - (sr.log() + mr)).abs().max().item() < 2e-3
    assert (tg - tr).abs().max().item() < 1e-3
    lse = sr.log() + mr
    g = torch.rand(M, device="cuda") * (labels != -100)
    dl = head_xent_grad(x, W, labels, lse, g, vocab_start)
    onehot = torch.zeros_like(logits)
    onehot[inside, local[inside]] = 1.0
    ref = ((logits - lse.unsqueeze(-1)).exp() - onehot) * g.unsqueeze(-1)
    assert (dl.float() - ref).abs().max().item() < 1e-2 * max(ref.abs().max().item(), 1e-3)
    torch.cuda.synchronize()
    assert _lib.read_error() is None


@pytest.mark.parametrize("M,hq,hk,dh,batch", [(512, 4, 2, 128, 2), (300, 2, 2, 64, 3), (8192, 32, 32, 128, 2)])
def test_qkv_projection_with_rotary_epilogue(M, hq, hk, dh, batch):
    """Packed QKV projection whose epilogue rotates the q and k heads, against the projection followed by the separate
    rotary kernel and against an fp32 reference."""
    from hetu_galvatron_b200.ops import functional as Fn
    from hetu_galvatron_b200.ops.gemm import RopeEpilogue
    torch.manual_seed(0)
    K = 512
    N = (hq + 2 * hk) * dh
    x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    W = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
    inv_freq = Fn.rope_inv_freq(dh, 10000.0, "cuda")
    fused = gemm(x, W, rope=RopeEpilogue((hq + hk) * dh, dh, inv_freq, None, batch, 0))
    plain = gemm(x, W)
    Fn.rope_(plain[:, : (hq + hk) * dh].view(M, hq + hk, dh), inv_freq, batch, 0, 0, None, False)
    assert (fused.float() - plain.float()).abs().max().item() < 3e-2 * plain.float().abs().max().item()
    # fp32 reference: rotation of the un-rounded projection
    y = x.float() @ W.float().t()
    pos = (torch.arange(M, device="cuda") // batch).float()
    ang = pos[:, None] * inv_freq[None, :]
    c, s_ = ang.cos(), ang.sin()
    yh = y[:, : (hq + hk) * dh].view(M, hq + hk, dh)
    a, b = yh[..., : dh // 2], yh[..., dh // 2:]
    ref = torch.cat([a * c[:, None] - b * s_[:, None], b * c[:, None] + a * s_[:, None]], -1).reshape(M, -1)
    assert (fused[:, : (hq + hk) * dh].float() - ref).abs().max().item() < 2e-2 * ref.abs().max().item()
    assert (fused[:, (hq + hk) * dh:].float() - y[:, (hq + hk) * dh:]).abs().max().item() < 2e-2 * y.abs().max().item()
    torch.cuda.synchronize()
    assert _lib.read_error() is None


@pytest.mark.parametrize("M,f,K", [(256, 128, 64), (300, 384, 256), (8192, 11008, 512), (512, 256, 4096)])
def test_up_projection_with_gated_activation_epilogue(M, f, K):
    """MLP up-projection whose epilogue also stores silu(gate) * up, against the projection followed by the separate
    SwiGLU kernel and an fp32 reference (single-CTA and pair kernels, by problem size)."""
    from hetu_galvatron_b200.ops import functional as Fn
    torch.manual_seed(0)
    x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    W = (torch.randn(2 * f, K, device="cuda") * (2.0 / K ** 0.5)).bfloat16()
    act = torch.empty(M, f, device="cuda", dtype=torch.bfloat16)
    gu = gemm(x, W, swiglu_out=act)
    plain = gemm(x, W)
    assert torch.equal(gu, plain)                       # the projection itself is stored as without the epilogue
    ref_act = Fn.swiglu_fwd(plain)
    assert (act.float() - ref_act.float()).abs().max().item() <= 2e-2 * ref_act.float().abs().max().item()
    y = x.float() @ W.float().t()
    ref32 = torch.nn.functional.silu(y[:, :f]) * y[:, f:]
    assert (act.float() - ref32).abs().max().item() < 3e-2 * ref32.abs().max().item()
    torch.cuda.synchronize()
    assert _lib.read_error() is None
