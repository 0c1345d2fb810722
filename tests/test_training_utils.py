"""Seeding, the data-parallel dataloader helper, loss printing and memory reporting (reference: galvatron/utils/
training_utils.py:7-40, memory_utils.py), single process."""
import random
from types import SimpleNamespace

import numpy as np
import torch

from hetu_galvatron_b200.core.dataloader import RandomTokenDataset, random_collate_fn
from hetu_galvatron_b200.utils import distributed_dataloader, memory_stats_mb, print_loss, print_peak_memory, set_seed


def test_set_seed_makes_every_generator_repeatable():
    set_seed(7)
    a = (random.random(), float(np.random.rand()), torch.rand(3))
    set_seed(7)
    b = (random.random(), float(np.random.rand()), torch.rand(3))
    assert a[0] == b[0] and a[1] == b[1] and torch.equal(a[2], b[2])
    set_seed(8)
    assert random.random() != a[0]


def test_dataloader_helper_and_random_dataset():
    ds = RandomTokenDataset(vocab_size=100, seq_length=16, dataset_size=64, seed=3)
    assert len(ds) == 64 and ds[0].shape == (17,) and int(ds.input_ids.max()) < 100
    # sentences of random length, zero padded
    lengths = (ds.input_ids != 0).sum(1)
    assert lengths.min() < 17 and (ds.input_ids[0][int(lengths[0]) + 1:] == 0).all()
    loader = distributed_dataloader(ds, global_bsz=8, shuffle=False, args=SimpleNamespace(pp_deg=1), collate_fn=random_collate_fn)
    tokens, labels = next(iter(loader))
    assert tokens.shape == (8, 16) and labels.shape == (8, 16) and torch.equal(tokens[:, 1:], labels[:, :-1])
    assert len(loader) == 8
    again = RandomTokenDataset(vocab_size=100, seq_length=16, dataset_size=64, seed=3)
    assert torch.equal(again.input_ids, ds.input_ids)


def test_loss_printing_and_memory_report(capsys):
    print_loss(SimpleNamespace(pp_deg=1), torch.tensor(2.5), 0, 3)
    print_loss(SimpleNamespace(pp_deg=1), [1.0, 2.0], 1, 4)
    print_loss(SimpleNamespace(pp_deg=1), None, 0, 5)
    out = capsys.readouterr().out.strip().splitlines()
    assert out == ["[Epoch 0] (Iteration 3): Loss = 2.500000", "[Epoch 1] (Iteration 4): Loss = 1.500000"]
    stats = memory_stats_mb()
    assert set(stats) == {"allocated", "max_allocated", "reserved", "max_reserved"}
    peak, cur = print_peak_memory("after step", None)
    assert peak >= cur >= 0 and "after step" in capsys.readouterr().out
