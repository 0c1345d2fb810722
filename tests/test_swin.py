"""Swin: windowed / shifted-window attention against a naive per-window restatement, patch merging order, and the
four-layer-type profile description."""
import math

import pytest
import torch

from hetu_galvatron_b200.models.swin import SwinLayerBlock, _relative_index, _shift_mask, model_layer_configs, swin_config, swin_specs
from hetu_galvatron_b200.models.transformer import LayerStrategy


def naive_window_attention(blk, qkv, b):
    """Loops over images, windows and heads with explicit index arithmetic."""
    R, ws, hl, dh, sh = blk.res, blk.ws, blk.heads_l, blk.dh, blk.shift
    x = qkv.view(R, R, b, 3, hl, dh)
    out = torch.zeros(R, R, b, hl, dh)
    table = blk.rel_table.detach()
    for n in range(b):
        for wy in range(R // ws):
            for wx in range(R // ws):
                # tokens of this window in the SHIFTED image -> their original coordinates
                coords = [((wy * ws + i + sh) % R, (wx * ws + j + sh) % R) for i in range(ws) for j in range(ws)]
                region = []
                for i in range(ws):
                    for j in range(ws):
                        y, xx = wy * ws + i, wx * ws + j                 # coordinates in the shifted image
                        ry = 0 if y < R - ws else (1 if y < R - sh else 2)
                        rx = 0 if xx < R - ws else (1 if xx < R - sh else 2)
                        region.append(ry * 3 + rx)
                for h in range(hl):
                    q = torch.stack([x[y, xx, n, 0, h] for (y, xx) in coords])
                    k = torch.stack([x[y, xx, n, 1, h] for (y, xx) in coords])
                    v = torch.stack([x[y, xx, n, 2, h] for (y, xx) in coords])
                    s = q @ k.t() / math.sqrt(dh)
                    for a in range(ws * ws):
                        for c in range(ws * ws):
                            dy = a // ws - c // ws + ws - 1
                            dx = a % ws - c % ws + ws - 1
                            s[a, c] += table[dy * (2 * ws - 1) + dx, h]
                            if sh and region[a] != region[c]:
                                s[a, c] = -1e9
                    o = torch.softmax(s, -1) @ v
                    for idx, (y, xx) in enumerate(coords):
                        out[y, xx, n, h] = o[idx]
    return out.reshape(R * R * b, hl * dh)


def test_window_attention_matches_naive():
    cfg = swin_config("swin-tiny-test", dtype=torch.float32)
    st = LayerStrategy()
    for stage, index in ((1, 0), (1, 1)):          # resolution 8, window 4: plain and shifted
        blk = SwinLayerBlock(cfg, st, stage, index, 3, False, torch.device("cpu"))
        with torch.no_grad():
            blk.rel_table.normal_(0, 0.5)
        b = 2
        torch.manual_seed(stage * 10 + index)
        qkv = torch.randn(blk.res * blk.res * b, 3 * blk.heads_l * blk.dh)
        got = blk._attention(qkv, b)
        ref = naive_window_attention(blk, qkv, b)
        assert (blk.shift > 0) == (index == 1)
        assert torch.allclose(got, ref, atol=1e-5), (got - ref).abs().max()


def test_relative_index_and_mask_shapes():
    idx = _relative_index(4)
    assert idx.shape == (16, 16) and int(idx.min()) == 0 and int(idx.max()) == 48 and int(idx[0, 0]) == 24
    m = _shift_mask(8, 4, 2)
    assert m.shape == (4, 16, 16) and float(m[0].abs().sum()) == 0 and float(m[3].min()) < 0


def test_four_layer_types_description():
    cfg = swin_config("swin-huge-patch4-window7-224")
    lc = model_layer_configs(cfg)
    assert [c["layer_num"] for c in lc] == [2, 2, 42, 2]
    assert [c["seq_len"] for c in lc] == [3136, 784, 196, 49]
    assert [c["hidden_size"] for c in lc] == [320, 640, 1280, 2560]
    specs = swin_specs(cfg)
    assert len([s for s in specs if s.layer_index is not None]) == 48 and specs[0].kind == "embed" and specs[-1].kind == "cls"


@pytest.mark.gpu
@pytest.mark.parametrize("stage,index", [(2, 0), (2, 1), (3, 0)])
def test_window_attention_on_the_kernels_matches_the_fp32_block(stage, index):
    """Swin-L blocks (windows of 12 x 12 tokens, head size 32) on the tcgen05 attention kernels with the additive bias /
    shift mask path, against the same block in fp32 on the CPU: output, input gradient, bias-table gradient."""
    from hetu_galvatron_b200.ops import _lib

    cfg_g = swin_config("swin-large-patch4-window12-384", dtype=torch.bfloat16)
    cfg_c = swin_config("swin-large-patch4-window12-384", dtype=torch.float32)
    st = LayerStrategy()
    blk_g = SwinLayerBlock(cfg_g, st, stage, index, 5, False, torch.device("cuda"))
    blk_c = SwinLayerBlock(cfg_c, st, stage, index, 5, False, torch.device("cpu"))
    with torch.no_grad():
        blk_c.rel_table.normal_(0, 0.5)
        blk_g.rel_table.copy_(blk_c.rel_table.to(torch.bfloat16))
        blk_c.rel_table.copy_(blk_g.rel_table.float())
    assert (blk_g.shift > 0) == (index == 1 and blk_g.ws < blk_g.res)
    b = 2
    torch.manual_seed(7)
    qkv_c = torch.randn(blk_c.res * blk_c.res * b, 3 * blk_c.heads_l * blk_c.dh).to(torch.bfloat16).float().requires_grad_(True)
    qkv_g = qkv_c.detach().to("cuda", torch.bfloat16).requires_grad_(True)
    out_c = blk_c._attention(qkv_c, b)
    out_g = blk_g._attention(qkv_g, b)
    dout = torch.randn_like(out_c).to(torch.bfloat16).float()
    gq_c, gt_c = torch.autograd.grad(out_c, [qkv_c, blk_c.rel_table], dout)
    gq_g, gt_g = torch.autograd.grad(out_g, [qkv_g, blk_g.rel_table], dout.to("cuda", torch.bfloat16))
    torch.cuda.synchronize()
    assert _lib.read_error() is None

    def rel(a, ref):
        return ((a.float().cpu() - ref).abs().max() / (ref.abs().max() + 1e-6)).item()

    assert rel(out_g, out_c) < 2e-2
    assert rel(gq_g, gq_c) < 3e-2
    assert rel(gt_g, gt_c) < 3e-2


def test_additive_terms_are_laid_out_for_the_kernels():
    """Bias (bf16, with its transpose for the backward kernel), additive mask (fp32) and group ids (int32, -1 padded) of a
    biased attention call: row stride a multiple of 64 covering both sequence lengths; the CPU restatement of the op treats
    group ids and the equivalent additive mask alike."""
    from hetu_galvatron_b200.ops import attention as at
    from hetu_galvatron_b200.ops import functional as Fn

    torch.manual_seed(0)
    h, s = 3, 49
    bias = torch.randn(h, s, s)
    ids = torch.randint(0, 3, (4, s), dtype=torch.int32)
    mask = torch.zeros(4, s, s).masked_fill(ids[:, :, None] != ids[:, None, :], -30000.0)
    add = at.Additive(s, s, bias, None, ids)
    assert add.ld == 64 and at.additive_ld(144, 144) == 192 and at.additive_ld(100, 200) == 256
    assert add.bias.shape == (h, s, 64) and add.bias.dtype == torch.bfloat16 and add.bias.is_contiguous()
    assert torch.equal(add.bias[:, :, :s], bias.to(torch.bfloat16)) and float(add.bias[:, :, s:].abs().max()) == 0.0
    assert torch.equal(add.bias_t[:, :, :s], bias.transpose(1, 2).to(torch.bfloat16))
    assert add.ids.dtype == torch.int32 and torch.equal(add.ids[:, :s], ids) and bool((add.ids[:, s:] == -1).all())
    m = at.Additive(s, s, None, mask, None)
    assert m.mask.dtype == torch.float32 and m.mask.shape == (4, s, 64) and m.bias is None
    q, k, v = (torch.randn(8, s, h, 16) for _ in range(3))
    a = Fn.biased_attention_reference(q, k, v, 0.25, bias, None, ids)
    b = Fn.biased_attention_reference(q, k, v, 0.25, bias, mask, None)
    assert torch.allclose(a, b, atol=1e-6)
    with pytest.raises(AssertionError):
        at.Additive(s, s + 1, None, None, ids)              # group ids need equal query and key lengths
