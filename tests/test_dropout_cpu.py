"""Hidden / embedding dropout with counter-based masks: the same elements are dropped under every tensor-parallel layout
and in the recomputed forward of a checkpointed block, so parallel runs reproduce the single-process losses with dropout
switched on (the reference forks a CUDA RNG tracker for this, models/gpt_hf/GPTModel_sequential.py:91-95)."""
import pytest
import torch

from dist_utils import run_worker
from hetu_galvatron_b200.models.transformer import BatchCtx, LayerStrategy, hidden_dropout

GPT = dict(hidden_size=64, num_heads=4, ffn_hidden_size=128, num_layers=4, vocab_size=250, seq_length=32)
BERT = dict(hidden_size=64, num_heads=4, ffn_hidden_size=128, num_layers=4, vocab_size=256, seq_length=32)
VIT = dict(hidden_size=64, num_heads=4, ffn_hidden_size=128, num_layers=4, image_size=32, patch_size=8, num_labels=16)
_BASE = {}


def _run(family, model, plan, world, p=0.1):
    return run_worker({"family": family, "model": dict(model, dropout=p), "plan": plan, "steps": 3}, world)


def _base(family, model, p=0.1):
    key = (family, p)
    if key not in _BASE:
        _BASE[key] = _run(family, model, dict(global_bsz=8, chunks=1), 1, p)
    return _BASE[key]


def _close(a, b, tol=2e-4):
    assert len(a) == len(b)
    for x, y in zip(a, b):
        assert abs(x - y) < tol * max(1.0, abs(y)), (a, b)


def test_mask_is_a_function_of_its_key():
    x = torch.ones(64, 32)
    ctx = BatchCtx(batch=2, seq=32, extra={"rng": (1234, 5, 0, 0)})
    full = LayerStrategy()
    y = hidden_dropout(x, 0.25, ctx, full, 7)
    kept = (y != 0).float().mean().item()
    assert abs(kept - 0.75) < 0.05 and torch.allclose(y[y != 0], torch.tensor(1 / 0.75))
    assert torch.equal(y, hidden_dropout(x, 0.25, ctx, full, 7))                          # same key, same mask
    assert not torch.equal(y, hidden_dropout(x, 0.25, ctx, full, 8))                      # another site
    assert not torch.equal(y, hidden_dropout(x, 0.25, BatchCtx(2, 32, extra={"rng": (1234, 6, 0, 0)}), full, 7))   # another step
    # a sequence-sharded activation takes its rows of the whole sequence's mask
    for r in range(2):
        st = LayerStrategy(tp=2, sp="megatron", tp_rank=r)
        assert torch.equal(hidden_dropout(x[r * 32:(r + 1) * 32], 0.25, ctx, st, 7), y[r * 32:(r + 1) * 32])
    assert hidden_dropout(x, 0.25, BatchCtx(2, 32), full, 7) is x                          # no key (evaluation): identity
    assert hidden_dropout(x, 0.0, ctx, full, 7) is x


def test_dropout_changes_the_loss():
    with_p, without = _base("gpt", GPT), _base("gpt", GPT, p=0.0)
    assert all(abs(a - b) > 1e-4 for a, b in zip(with_p, without))


@pytest.mark.parametrize("plan", [dict(global_bsz=8, global_tp_deg=2, vocab_tp=2),
                                  dict(global_bsz=8, global_tp_deg=2, vocab_tp=2, sequence_parallel=True)], ids=["tp2", "tp2_sp"])
def test_gpt_tensor_parallel_layouts_drop_the_same_elements(plan):
    _close(_run("gpt", GPT, plan, 2), _base("gpt", GPT))


def test_checkpoint_recompute_sees_the_same_masks():
    _close(_run("gpt", GPT, dict(global_bsz=8, chunks=1, global_checkpoint=1), 1), _base("gpt", GPT))


def test_bert_post_ln_and_vit_embedding_dropout_under_tp():
    _close(_run("bert", BERT, dict(global_bsz=8, global_tp_deg=2, vocab_tp=2, sequence_parallel=True), 2), _base("bert", BERT))
    _close(_run("vit", VIT, dict(global_bsz=8, global_tp_deg=2, vocab_tp=2), 2), _base("vit", VIT))


def test_swin_drop_path_is_the_same_under_tensor_parallelism_and_recomputation():
    """Stochastic depth of the Swin attention branch (reference: models/swin/SwinModel_tensor_parallel.py:63,76): whole samples
    drop out of a block, the draw is keyed like the dropout masks, so TP = 2 and a checkpointed (recomputed) run reproduce the
    single-process losses; evaluation and rate 0 leave the model as it was."""
    swin = dict(model_size="swin-tiny-test")
    run = lambda model, plan, world: run_worker({"family": "swin", "model": model, "plan": plan, "steps": 3}, world)
    off = run(swin, dict(global_bsz=8, chunks=1), 1)
    on = run(dict(swin, drop_path_rate=0.3), dict(global_bsz=8, chunks=1), 1)
    assert all(abs(a - b) > 1e-5 for a, b in zip(on, off))
    _close(run(dict(swin, drop_path_rate=0.3), dict(global_bsz=8, global_tp_deg=2, vocab_tp=2), 2), on, tol=2e-5)
    _close(run(dict(swin, drop_path_rate=0.3), dict(global_bsz=8, chunks=1, global_checkpoint=1), 1), on, tol=2e-5)


def test_swin_flags_reach_the_config():
    from types import SimpleNamespace

    from hetu_galvatron_b200.models.arguments import config_from_args

    base = dict(model_size="swin-tiny-test", image_size=None, patch_size=None, depths=None, embed_dim=None, window_size=None,
                num_heads=None, mlp_ratio=None, num_classes=None, num_labels=1000, num_channels=3, drop_path_rate=None,
                set_model_config_manually=0, set_layernum_manually=0, set_seqlen_manually=0)
    cfg, _ = config_from_args("swin", SimpleNamespace(**dict(base, model_size="swin-large-patch4-window12-384")), torch.float32)
    assert cfg.drop_path_rate == 0.1                         # the training programs take the model size's rate by default
    cfg, _ = config_from_args("swin", SimpleNamespace(**dict(base, drop_path_rate=0.0)), torch.float32)
    assert cfg.drop_path_rate == 0.0
    manual = dict(base, set_model_config_manually=1, embed_dim=48, num_heads=[2, 4, 8, 16], mlp_ratio=2, num_classes=10,
                  depths=[1, 1, 2, 1], window_size=4)
    cfg, specs = config_from_args("swin", SimpleNamespace(**manual), torch.float32)
    assert (cfg.embed_dim, cfg.stage_heads, cfg.mlp_ratio, cfg.num_labels, cfg.depths, cfg.window_size) == \
        (48, [2, 4, 8, 16], 2, 10, [1, 1, 2, 1], 4)
    assert cfg.hidden_size == 48 and cfg.ffn_hidden_size == 96 and cfg.num_layers == 5
    assert len([s for s in specs if s.layer_index is not None]) == 5
