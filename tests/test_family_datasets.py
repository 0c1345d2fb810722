"""Random datasets of every family (reference: galvatron/models/<family>/dataloader.py) and their collate functions: shapes,
masking rules, and one training step of the family's model on a collated batch."""
from types import SimpleNamespace

import pytest
import torch

from hetu_galvatron_b200.core.hybrid_model import construct_hybrid_parallel_model
from hetu_galvatron_b200.core.plan import HybridPlan
from hetu_galvatron_b200.models import build_model_specs
from hetu_galvatron_b200.models import dataloader as D
from hetu_galvatron_b200.utils.training_utils import distributed_dataloader


def test_decoder_sentences_are_padded_behind_their_length():
    args = SimpleNamespace(vocab_size=100, seq_length=16, seed=7)
    ds = D.DataLoaderForLlama(args, None, 64)
    assert len(ds) == 64 and ds[0].shape == (17,)
    for i in range(64):
        n = int(ds.lengths[i])
        assert 1 <= n <= 16 and bool((ds[i][n + 1:] == 0).all())
    ids, labels = D.random_collate_fn([ds[i] for i in range(4)])
    assert ids.shape == labels.shape == (4, 16) and torch.equal(ids[:, 1:], labels[:, :-1])
    assert torch.equal(D.DataLoaderForGPT(args, None, 64).input_ids, ds.input_ids)        # same arguments, same samples


def test_bert_pairs_and_masking():
    args = SimpleNamespace(vocab_size=1000, seq_length=64, seed=3)
    ds = D.DataLoaderForBert(args, None, 256)
    ids, labels, extra = D.random_collate_fn_bert([ds[i] for i in range(256)])
    mask, types = extra["attention_mask"], extra["token_type_ids"]
    assert ids.shape == labels.shape == mask.shape == types.shape == (256, 64)
    n = mask.sum(1)
    assert bool((ids[:, 0] == ds.CLS).all()) and bool((ids[torch.arange(256), n - 1] == ds.SEP).all())
    assert bool(((ids == ds.PAD) | (mask == 1)).all()) and bool((labels[mask == 0] == D.IGNORE).all())
    assert bool((types[mask == 0] == 0).all()) and bool((types.sum(1) > 0).all())           # both sentences present
    chosen = labels != D.IGNORE
    frac = chosen.sum().item() / ((mask == 1).sum().item() - 3 * 256)
    assert 0.11 < frac < 0.19                                                               # 15 % of the ordinary tokens
    masked = (ids == ds.MASK) & chosen
    assert 0.7 < masked.sum().item() / chosen.sum().item() < 0.9                            # 80 % of them show [MASK]
    assert not bool((labels[chosen] == ds.MASK).any())                                      # labels keep the original ids
    kept = chosen & (ids == labels)
    assert 0.03 < kept.sum().item() / chosen.sum().item() < 0.2


def test_t5_sides_have_their_own_lengths():
    args = SimpleNamespace(vocab_size=200, seq_length=16, encoder_seq_length=16, decoder_seq_length=8, seed=5)
    ds = D.DataLoaderForT5(args, None, 32)
    enc, labels, extra = D.random_collate_fn_t5([ds[i] for i in range(32)])
    assert enc.shape == (32, 16) and labels.shape == extra["decoder_input_ids"].shape == (32, 8)
    assert bool((extra["decoder_input_ids"][:, 0] == 0).all())
    dm = extra["decoder_attention_mask"]
    assert bool((labels[dm == 0] == D.IGNORE).all()) and bool((labels[dm == 1] > 0).all())
    # teacher forcing: the decoder sees the target shifted right
    assert torch.equal(extra["decoder_input_ids"][:, 1:][dm[:, 1:] == 1], labels[:, :-1][dm[:, 1:] == 1])


def test_images():
    args = SimpleNamespace(image_size=32, num_channels=3, num_labels=10, seed=1)
    ds = D.DataLoaderForViT(args, None, 16)
    px, lb = D.vit_collate_fn([ds[i] for i in range(4)])
    assert px.shape == (4, 3, 32, 32) and lb.shape == (4,) and int(lb.max()) < 10
    assert torch.equal(ds[3][0], D.DataLoaderForSwin(args, None, 16)[3][0])
    assert D.random_dataset("vit_hf", args, None, 8)[1] is D.vit_collate_fn


FAMILIES = {
    "llama": dict(hidden_size=32, num_heads=2, num_kv_heads=2, ffn_hidden_size=64, num_layers=2, vocab_size=128, seq_length=16),
    "gpt": dict(hidden_size=32, num_heads=2, ffn_hidden_size=64, num_layers=2, vocab_size=128, seq_length=16),
    "bert": dict(hidden_size=32, num_heads=2, ffn_hidden_size=64, num_layers=2, vocab_size=128, seq_length=16),
    "t5": dict(hidden_size=32, num_heads=2, ffn_hidden_size=64, num_layers=1, num_decoder_layers=1, vocab_size=128, seq_length=16,
               decoder_seq_length=8),
    "vit": dict(hidden_size=32, num_heads=2, ffn_hidden_size=64, num_layers=2, image_size=16, patch_size=4, num_labels=8),
    "swin": dict(model_size="swin-tiny-test"),
}


@pytest.mark.parametrize("family", list(FAMILIES))
def test_a_loader_feeds_the_family_model(family):
    cfg, specs = build_model_specs(family, dtype=torch.float32, **FAMILIES[family])
    n_layers = len([s for s in specs if s.layer_index is not None])
    model = construct_hybrid_parallel_model(cfg, HybridPlan.from_global(n_layers, 1, global_bsz=4, chunks=2), specs, torch.device("cpu"))
    args = SimpleNamespace(vocab_size=cfg.vocab_size, seq_length=cfg.seq_length, decoder_seq_length=getattr(cfg, "decoder_seq_length", None),
                           image_size=cfg.image_size, num_channels=cfg.num_channels, num_labels=cfg.num_labels, seed=11)
    ds, collate = D.random_dataset(family, args, None, 16)
    loader = distributed_dataloader(ds, 4, shuffle=False, collate_fn=collate, model=model)
    losses = []
    for it, batch in zip(range(2), loader):
        if family in ("vit", "swin"):
            batch = (batch[0].to(cfg.dtype), batch[1])
        loss = model.forward_backward(batch, it)
        model.optimizer_step(1e-3)
        model.zero_grad()
        losses.append(float(loss))
    assert all(0.0 < v < 10.0 for v in losses)


def test_sampler_follows_the_data_layout_of_the_model():
    """Two tensor-parallel ranks of one data-parallel position draw the same samples; the other position draws the rest."""
    args = SimpleNamespace(vocab_size=100, seq_length=8, seed=2)
    ds = D.DataLoaderForLlama(args, None, 16)

    def rows(lo):
        fake = SimpleNamespace(local_batch_size=lambda: 2, batch_slice=lambda: (lo, lo + 2))
        return [b[0] for b in distributed_dataloader(ds, 4, shuffle=False, collate_fn=D.random_collate_fn, model=fake)]

    first, again, second = rows(0), rows(0), rows(2)
    assert len(first) == 4 and all(b.shape == (2, 8) for b in first)
    assert all(torch.equal(a, b) for a, b in zip(first, again))
    seen = torch.cat(first + second)
    assert len({tuple(r.tolist()) for r in seen}) == 16                   # together they cover the dataset once
