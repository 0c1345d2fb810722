"""HBM-bound kernels (norms, RoPE, activations, embedding, cross entropy, AdamW) vs PyTorch fp32."""

import pytest
import torch

from hetu_galvatron_b200.ops import functional as Fn

pytestmark = pytest.mark.gpu
DEV = "cuda"


def close(a, b, tol=2e-2):
    a, b = a.float(), b.float()
    denom = b.abs().max().item() + 1e-6
    assert (a - b).abs().max().item() / denom < tol, (a - b).abs().max().item() / denom


@pytest.mark.parametrize("rows,cols", [(7, 256), (300, 4096), (64, 5120), (33, 1280), (5, 8192)])
def test_rmsnorm(rows, cols):
    torch.manual_seed(0)
    x = torch.randn(rows, cols, device=DEV, dtype=torch.bfloat16)
    r = torch.randn(rows, cols, device=DEV, dtype=torch.bfloat16)
    w = (1 + 0.1 * torch.randn(cols, device=DEV)).bfloat16()
    y, h, rstd = Fn.rmsnorm_fwd(x, w, 1e-5, r)
    yr, hr, rr = Fn.rmsnorm_fwd(x.cpu().float(), w.cpu().float(), 1e-5, r.cpu().float())
    close(y.cpu(), yr)
    close(h.cpu(), hr)
    close(rstd.cpu(), rr, 1e-2)
    dy = torch.randn(rows, cols, device=DEV, dtype=torch.bfloat16)
    dres = torch.randn(rows, cols, device=DEV, dtype=torch.bfloat16)
    dw = torch.zeros(cols, device=DEV)
    dx = Fn.rmsnorm_bwd(dy, h, w, rstd, dres, dw)
    dwr = torch.zeros(cols)
    dxr = Fn.rmsnorm_bwd(dy.cpu().float(), h.cpu().float(), w.cpu().float(), rstd.cpu(), dres.cpu().float(), dwr)
    close(dx.cpu(), dxr)
    close(dw.cpu(), dwr)


def test_norm_weight_gradients_are_bitwise_repeatable():
    """The weight (and bias) gradient is reduced in two stages in a fixed order, without atomics: same bits every run."""
    torch.manual_seed(1)
    rows, cols = 8192, 4096
    x = torch.randn(rows, cols, device=DEV, dtype=torch.bfloat16)
    w = (1 + 0.1 * torch.randn(cols, device=DEV)).bfloat16()
    dy = torch.randn(rows, cols, device=DEV, dtype=torch.bfloat16)
    _, _, rstd = Fn.rmsnorm_fwd(x, w, 1e-5)
    outs = []
    for _ in range(3):
        dw = torch.zeros(cols, device=DEV)
        Fn.rmsnorm_bwd(dy, x, w, rstd, None, dw)
        outs.append(dw.clone())
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    b = torch.zeros(cols, device=DEV, dtype=torch.bfloat16)
    _, _, mean, rstd = Fn.layernorm_fwd(x, w, b, 1e-5)
    outs = []
    for _ in range(2):
        dw, db = torch.zeros(cols, device=DEV), torch.zeros(cols, device=DEV)
        Fn.layernorm_bwd(dy, x, w, mean, rstd, None, dw, db)
        outs.append((dw.clone(), db.clone()))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    # accumulation semantics: a second call adds to what is there
    dw2 = outs[0][0].clone()
    Fn.layernorm_bwd(dy, x, w, mean, rstd, None, dw2, torch.zeros(cols, device=DEV))
    close(dw2, 2 * outs[0][0], 1e-3)


@pytest.mark.parametrize("rows,cols", [(9, 768), (257, 1280), (40, 4096)])
def test_layernorm(rows, cols):
    torch.manual_seed(0)
    x = torch.randn(rows, cols, device=DEV, dtype=torch.bfloat16) + 0.5
    w = (1 + 0.1 * torch.randn(cols, device=DEV)).bfloat16()
    b = (0.1 * torch.randn(cols, device=DEV)).bfloat16()
    y, h, mean, rstd = Fn.layernorm_fwd(x, w, b, 1e-5)
    yr = torch.nn.functional.layer_norm(x.float(), (cols,), w.float(), b.float(), 1e-5)
    close(y, yr)
    dy = torch.randn(rows, cols, device=DEV, dtype=torch.bfloat16)
    dw = torch.zeros(cols, device=DEV)
    db = torch.zeros(cols, device=DEV)
    dx = Fn.layernorm_bwd(dy, h, w, mean, rstd, None, dw, db)
    xr = x.float().requires_grad_(True)
    wr = w.float().requires_grad_(True)
    br = b.float().requires_grad_(True)
    torch.nn.functional.layer_norm(xr, (cols,), wr, br, 1e-5).backward(dy.float())
    close(dx, xr.grad)
    close(dw, wr.grad)
    close(db, br.grad)


def test_rope_roundtrip_and_reference():
    torch.manual_seed(0)
    tokens, hq, hk, dh, seq = 512, 8, 2, 128, 256
    qkv = torch.randn(tokens, (hq + 2 * hk) * dh, device=DEV, dtype=torch.bfloat16)
    ref = qkv.clone().cpu().float()
    inv = Fn.rope_inv_freq(dh, 10000.0, DEV)
    q = qkv[:, : hq * dh].view(tokens, hq, dh)
    k = qkv[:, hq * dh:(hq + hk) * dh].view(tokens, hk, dh)
    Fn.rope_(q, inv, 1, seq, 3)
    Fn.rope_(k, inv, 1, seq, 3)
    qr = ref[:, : hq * dh].view(tokens, hq, dh)
    kr = ref[:, hq * dh:(hq + hk) * dh].view(tokens, hk, dh)
    Fn.rope_(qr, inv.cpu(), 1, seq, 3)
    Fn.rope_(kr, inv.cpu(), 1, seq, 3)
    close(qkv.cpu(), ref)
    # inverse rotation restores the input up to bf16 rounding
    orig = ref.clone()
    Fn.rope_(q, inv, 1, seq, 3, inverse=True)
    Fn.rope_(qr, inv.cpu(), 1, seq, 3, inverse=True)
    close(qkv.cpu(), ref)


def test_swiglu_gelu_colsum():
    torch.manual_seed(0)
    gu = torch.randn(300, 2 * 1376, device=DEV, dtype=torch.bfloat16)
    out = Fn.swiglu_fwd(gu)
    close(out, Fn.swiglu_fwd(gu.cpu().float()).to(DEV))
    d = torch.randn_like(out)
    close(Fn.swiglu_bwd(d, gu), Fn.swiglu_bwd(d.cpu().float(), gu.cpu().float()).to(DEV))
    x = torch.randn(128, 1024, device=DEV, dtype=torch.bfloat16)
    close(Fn.gelu_fwd(x), Fn.gelu_fwd(x.cpu().float()).to(DEV))
    dy = torch.randn_like(x)
    close(Fn.gelu_bwd(dy, x), Fn.gelu_bwd(dy.cpu().float(), x.cpu().float()).to(DEV))
    acc = torch.zeros(1024, device=DEV)
    big = torch.randn(4099, 1024, device=DEV, dtype=torch.bfloat16)
    Fn.colsum_accum(big, acc)
    close(acc, big.float().sum(0), 1e-2)


def test_embedding():
    torch.manual_seed(0)
    V, H = 1000, 512
    table = torch.randn(V, H, device=DEV, dtype=torch.bfloat16)
    pos = torch.randn(128, H, device=DEV, dtype=torch.bfloat16)
    ids = torch.randint(0, 2 * V, (4, 128), device=DEV)
    pid = torch.arange(128, device=DEV).repeat(4, 1)
    out = Fn.embedding_fwd(ids, table, 0, pid, pos)
    ref = Fn.embedding_fwd(ids.cpu(), table.cpu().float(), 0, pid.cpu(), pos.cpu().float())
    close(out.cpu(), ref)
    dt = torch.zeros(V, H, device=DEV)
    dout = torch.randn(4, 128, H, device=DEV, dtype=torch.bfloat16)
    Fn.embedding_bwd(ids, dout, dt, 0)
    dtr = torch.zeros(V, H)
    Fn.embedding_bwd(ids.cpu(), dout.cpu().float(), dtr, 0)
    close(dt.cpu(), dtr)


@pytest.mark.parametrize("V", [1000, 32000, 1031 * 8])
def test_cross_entropy(V):
    torch.manual_seed(0)
    rows = 257
    logits = (torch.randn(rows, V, device=DEV) * 3).bfloat16()
    labels = torch.randint(0, V, (rows,), device=DEV)
    labels[5] = -100
    lf = logits.float().clone().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(lf, labels, reduction="none", ignore_index=-100)
    ref.sum().backward()
    mx, se, tg = Fn.xent_stats(logits, labels)
    loss = Fn.xent_loss_grad_(logits, labels, mx, se, tg, 1.0)
    close(loss, ref, 1e-2)
    close(logits, lf.grad, 2e-2)


def test_adamw_and_sumsq():
    torch.manual_seed(0)
    n = 100003
    master = torch.randn(n, device=DEV)
    m = torch.zeros(n, device=DEV)
    v = torch.zeros(n, device=DEV)
    param = master.bfloat16()
    ref_p = torch.nn.Parameter(master.clone())
    opt = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in range(1, 4):
        g = torch.randn(n, device=DEV)
        ref_p.grad = g.clone()
        opt.step()
        Fn.adamw_step_(master, m, v, g, param, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step)
    close(master, ref_p.data, 1e-4)
    close(param, ref_p.data, 1e-2)
    out = torch.zeros(1, device=DEV)
    gb = torch.randn(n, device=DEV).bfloat16()
    Fn.sumsq_accum(gb, out)
    assert abs(out.item() - gb.float().pow(2).sum().item()) / out.item() < 1e-3
