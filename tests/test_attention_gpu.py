"""tcgen05 flash attention forward/backward vs an fp32 PyTorch reference."""
import math

import pytest
import torch

from hetu_galvatron_b200.ops import functional as Fn
from hetu_galvatron_b200.ops import _lib

pytestmark = pytest.mark.gpu

CASES = [
    # b, sq, sk, hq, hk, dh, causal
    (1, 128, 128, 2, 2, 128, True),
    (2, 256, 256, 4, 2, 128, True),
    (1, 200, 200, 2, 2, 128, True),
    (1, 257, 257, 4, 4, 80, False),
    (2, 256, 256, 4, 4, 50, True),      # head size not a multiple of 8: zero-padded onto the kernel
    (2, 384, 384, 4, 4, 64, True),
    (1, 128, 384, 2, 1, 128, True),
    (1, 1024, 1024, 8, 8, 128, True),
    (1, 320, 320, 2, 2, 128, False),
    (1, 64, 64, 2, 2, 32, True),
]


def _mk(b, sq, sk, hq, hk, dh):
    torch.manual_seed(0)
    # q, k, v as views of one packed projection output, like the model produces them
    tot = (hq + 2 * hk) * dh
    if sq == sk:
        qkv = torch.randn(b, sq, tot, device="cuda", dtype=torch.bfloat16)
        q = qkv[..., : hq * dh].view(b, sq, hq, dh)
        k = qkv[..., hq * dh:(hq + hk) * dh].view(b, sk, hk, dh)
        v = qkv[..., (hq + hk) * dh:].view(b, sk, hk, dh)
    else:
        q = torch.randn(b, sq, hq, dh, device="cuda", dtype=torch.bfloat16)
        k = torch.randn(b, sk, hk, dh, device="cuda", dtype=torch.bfloat16)
        v = torch.randn(b, sk, hk, dh, device="cuda", dtype=torch.bfloat16)
    return q, k, v


def _rel(a, b):
    return ((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-6)).item()


@pytest.mark.parametrize("b,sq,sk,hq,hk,dh,causal", CASES)
def test_attention_fwd(b, sq, sk, hq, hk, dh, causal):
    q, k, v = _mk(b, sq, sk, hq, hk, dh)
    scale = 1.0 / math.sqrt(dh)
    o, lse = Fn.attention_fwd(q, k, v, causal, scale)
    torch.cuda.synchronize()
    assert _lib.read_error() is None
    o_ref, lse_ref = Fn.attention_reference(q.float(), k.float(), v.float(), causal, scale)
    assert _rel(o, o_ref) < 2e-2
    assert (lse - lse_ref).abs().max().item() < 2e-2


@pytest.mark.parametrize("b,sq,sk,hq,hk,dh,causal", CASES)
def test_attention_bwd(b, sq, sk, hq, hk, dh, causal):
    q, k, v = _mk(b, sq, sk, hq, hk, dh)
    scale = 1.0 / math.sqrt(dh)
    o, lse = Fn.attention_fwd(q, k, v, causal, scale)
    dout = torch.randn_like(o)
    dq, dk, dv = Fn.attention_bwd(dout, q, k, v, o, lse, causal, scale)
    torch.cuda.synchronize()
    assert _lib.read_error() is None
    qf, kf, vf = (t.float().detach().clone().requires_grad_(True) for t in (q, k, v))
    o_ref, _ = Fn.attention_reference(qf, kf, vf, causal, scale)
    o_ref.backward(dout.float())
    assert _rel(dq, qf.grad) < 3e-2
    assert _rel(dk, kf.grad) < 3e-2
    assert _rel(dv, vf.grad) < 3e-2


def test_attention_is_repeatable():
    """Forward, dK and dV have a fixed accumulation order (bitwise equal across runs); dQ is summed over KV tiles by
    fp32 reduce-adds whose order depends on CTA scheduling, so it is only equal up to fp32 rounding."""
    q, k, v = _mk(2, 1024, 1024, 8, 2, 128)
    scale = 1.0 / math.sqrt(128)
    o1, lse1 = Fn.attention_fwd(q, k, v, True, scale)
    o2, lse2 = Fn.attention_fwd(q, k, v, True, scale)
    assert torch.equal(o1, o2) and torch.equal(lse1, lse2)
    dout = torch.randn_like(o1)
    dq1, dk1, dv1 = Fn.attention_bwd(dout, q, k, v, o1, lse1, True, scale)
    dq2, dk2, dv2 = Fn.attention_bwd(dout, q, k, v, o1, lse1, True, scale)
    torch.cuda.synchronize()
    assert torch.equal(dk1, dk2) and torch.equal(dv1, dv2)
    assert _rel(dq1, dq2) < 1e-2
    assert _lib.read_error() is None


@pytest.mark.parametrize("b,s,hq,hk,dh,causal,lens", [
    (3, 384, 4, 2, 128, False, [384, 200, 65]),       # whole padded tiles, a ragged tile, a full sequence
    (2, 320, 2, 2, 64, True, [129, 320]),             # decoder padding on top of the causal mask
    (2, 256, 4, 4, 128, False, [1, 128]),             # a single real key; a length on a tile boundary
])
def test_attention_key_lengths(b, s, hq, hk, dh, causal, lens):
    """Per-sequence key lengths (padding masks): padded keys take no part in the softmax, their dK / dV are zero."""
    q, k, v = _mk(b, s, s, hq, hk, dh)
    scale = 1.0 / math.sqrt(dh)
    kv_lens = torch.tensor(lens, device="cuda", dtype=torch.int32)
    o, lse = Fn.attention_fwd(q, k, v, causal, scale, kv_lens=kv_lens)
    do = torch.randn_like(o)
    dq, dk, dv = Fn.attention_bwd(do, q, k, v, o, lse, causal, scale, kv_lens=kv_lens)
    torch.cuda.synchronize()
    assert _lib.read_error() is None
    qf, kf, vf = (t.float().clone().requires_grad_(True) for t in (q, k, v))
    o_ref, lse_ref = Fn.attention_reference(qf, kf, vf, causal, scale, kv_lens)
    # rows whose causal window holds no real key cannot occur here (every length >= 1 and key 0 is always visible)
    (o_ref * do.float()).sum().backward()
    assert _rel(o, o_ref) < 2e-2 and (lse - lse_ref).abs().max().item() < 2e-2
    assert _rel(dq, qf.grad) < 3e-2 and _rel(dk, kf.grad) < 3e-2 and _rel(dv, vf.grad) < 3e-2
    for i, n in enumerate(lens):
        assert dk[i, n:].abs().max().item() == 0 if n < s else True
        assert dv[i, n:].abs().max().item() == 0 if n < s else True


@pytest.mark.parametrize("b,s,hq,hk,dh,causal", [(2, 256, 4, 2, 128, True), (1, 200, 2, 2, 64, False)])
def test_attention_dropout_matches_reference_mask(b, s, hq, hk, dh, causal):
    """Dropout of the attention probabilities: the kernels draw the mask from (seed, batch, head, q, k); the fp32
    reference draws the same mask in PyTorch, so outputs and gradients must agree, forward and backward."""
    q, k, v = _mk(b, s, s, hq, hk, dh)
    scale = 1.0 / math.sqrt(dh)
    drop = (0.25, 0x1234ABCD5678EF01, 5)
    o, lse = Fn.attention_fwd(q, k, v, causal, scale, dropout=drop)
    o2, _ = Fn.attention_fwd(q, k, v, causal, scale, dropout=drop)
    assert torch.equal(o, o2)                                  # same seed, same mask
    o3, _ = Fn.attention_fwd(q, k, v, causal, scale, dropout=(0.25, 7, 5))
    assert not torch.equal(o, o3)
    do = torch.randn_like(o)
    dq, dk, dv = Fn.attention_bwd(do, q, k, v, o, lse, causal, scale, dropout=drop)
    torch.cuda.synchronize()
    assert _lib.read_error() is None
    qf, kf, vf = (t.float().clone().requires_grad_(True) for t in (q, k, v))
    o_ref, lse_ref = Fn.attention_reference(qf, kf, vf, causal, scale, None, drop)
    (o_ref * do.float()).sum().backward()
    assert _rel(o, o_ref) < 2e-2 and (lse - lse_ref).abs().max().item() < 2e-2
    assert _rel(dq, qf.grad) < 3e-2 and _rel(dk, kf.grad) < 3e-2 and _rel(dv, vf.grad) < 3e-2
    keep = Fn.dropout_keep_mask(0.25, drop[1], b, hq, s, s, 5, "cuda").float().mean().item()
    assert abs(keep - 0.75) < 0.01


@pytest.mark.parametrize("b,s,h,dh,mask_n,with_bias,kind", [
    (6, 144, 3, 32, 3, True, "ids"),      # Swin-L windows: 12 x 12 tokens, shifted (region ids per window position)
    (4, 144, 6, 32, 0, True, None),       # un-shifted block: relative-position bias only
    (8, 49, 4, 32, 4, True, "ids"),       # 7 x 7 windows: a single partial tile, row stride padded to 64
    (2, 200, 2, 64, 2, False, "ids"),     # ids only, rows that are not a multiple of the tile sizes
    (6, 144, 3, 32, 3, True, "mask"),     # the general additive mask
    (2, 200, 2, 64, 2, False, "mask"),
    (3, 144, 2, 128, 1, True, "mask"),
])
def test_attention_with_bias_mask_and_group_ids(b, s, h, dh, mask_n, with_bias, kind):
    """Windowed attention: additive bias per head, and per (batch element % mask_n) either group ids or an additive mask;
    forward and every gradient (the bias gradient is summed over the batch inside the backward kernel) against fp32
    PyTorch expressions."""
    from hetu_galvatron_b200.ops import autograd as A

    torch.manual_seed(1)
    q, k, v = (torch.randn(b, s, h, dh, device="cuda", dtype=torch.bfloat16, requires_grad=True) for _ in range(3))
    bias = (torch.randn(h, s, s, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True) if with_bias else None
    mask = ids = None
    if kind == "mask":
        blocked = torch.rand(mask_n, s, s, device="cuda") < 0.3
        blocked[:, torch.arange(s), torch.arange(s)] = False          # every row keeps at least its own key
        mask = torch.zeros(mask_n, s, s, device="cuda", dtype=torch.bfloat16).masked_fill(blocked, -30000.0)
    elif kind == "ids":
        ids = torch.randint(0, 4, (mask_n, s), device="cuda", dtype=torch.int32)
    scale = 1.0 / math.sqrt(dh)
    o = A.biased_attention(q, k, v, bias, mask, ids, scale)
    do = torch.randn_like(o)
    grads = torch.autograd.grad(o, [t for t in (q, k, v, bias) if t is not None], do)
    torch.cuda.synchronize()
    assert _lib.read_error() is None
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    bf = bias.detach().float().requires_grad_(True) if with_bias else None
    o_ref = Fn.biased_attention_reference(qf, kf, vf, scale, bf, mask, ids)
    ref = torch.autograd.grad(o_ref, [t for t in (qf, kf, vf, bf) if t is not None], do.float())
    assert _rel(o, o_ref) < 2e-2
    for got, want in zip(grads, ref):
        assert got.shape == want.shape and _rel(got, want) < 3e-2
    # invisible entries carry no probability: the bias gradient there is exactly zero
    if with_bias and mask_n == 1 and kind == "mask":
        assert grads[3].float()[:, mask[0] < -1.0].abs().max().item() == 0.0
    if with_bias and kind == "ids":
        hidden = (ids[:, :, None] != ids[:, None, :]).all(dim=0)       # hidden in every window position
        if hidden.any():
            assert grads[3].float()[:, hidden].abs().max().item() == 0.0
