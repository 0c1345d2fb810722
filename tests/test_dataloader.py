"""Indexed token datasets: file format round trip, sample index against a plain numpy restatement, epoch coverage,
blending proportions, the per-rank batch iterator (reference test: tests/models/test_dataloader.py)."""
import numpy as np
import pytest
import torch

from hetu_galvatron_b200.core import dataloader as D


@pytest.fixture()
def corpus(tmp_path):
    rng = np.random.RandomState(0)
    docs = [rng.randint(1, 1000, size=rng.randint(3, 40)).tolist() for _ in range(50)]
    prefix = str(tmp_path / "corpus")
    D.write_indexed_dataset(prefix, docs)
    return prefix, docs


def test_indexed_dataset_round_trip(corpus):
    prefix, docs = corpus
    data = D.IndexedDataset(prefix)
    assert len(data) == len(docs)
    for i in (0, 7, 49):
        assert data.document(i).tolist() == docs[i]


def test_samples_are_windows_of_the_shuffled_stream(corpus):
    prefix, docs = corpus
    data = D.IndexedDataset(prefix)
    seq = 16
    ds = D.GPTTokenDataset(data, (0, 40), seq, num_samples=100, seed=3)
    stream = np.concatenate([np.asarray(docs[d]) for d in ds.doc_idx])
    assert len(ds) == (len(stream) - 1) // seq
    for i in (0, 1, 17, len(ds) - 1):
        s = int(ds.shuffle_idx[i])
        assert ds[i].tolist() == stream[s * seq:(s + 1) * seq + 1].tolist()
    # every epoch visits every document of the split exactly once
    per_epoch = ds.doc_idx.reshape(-1, 40)
    for row in per_epoch:
        assert sorted(row.tolist()) == list(range(40))
    # determinism
    ds2 = D.GPTTokenDataset(data, (0, 40), seq, num_samples=100, seed=3)
    assert np.array_equal(ds.shuffle_idx, ds2.shuffle_idx) and np.array_equal(ds.sample_idx, ds2.sample_idx)


def test_split_ranges_and_blending(corpus, tmp_path):
    assert D.split_ranges(1000, "969,30,1") == [(0, 969), (969, 999), (999, 1000)]
    prefix, docs = corpus
    other = str(tmp_path / "other")
    D.write_indexed_dataset(other, [[5000 + i] * 20 for i in range(30)])
    ds = D.build_dataset(["0.75", prefix, "0.25", other], 8, 400, seed=1, split="100,0,0")
    out = np.empty((400, 9), dtype=np.int64)
    ds.gather(np.arange(400), out, threads=4)
    frac = float((out[:, 0] >= 5000).mean())
    assert abs(frac - 0.25) < 0.02
    w, idx = ds.which, ds.index
    assert idx[w == 0].tolist() == list(range(int((w == 0).sum())))


def test_iterator_slices_global_batch(corpus):
    prefix, _ = corpus
    ds = D.build_dataset([prefix], 8, 64, seed=5, split="100,0,0")
    full = D.TokenBatchIterator(ds, 8, 0, 8, torch.device("cpu"))
    part = D.TokenBatchIterator(ds, 8, 4, 8, torch.device("cpu"))
    for _ in range(3):
        tf, lf = next(full)
        tp, lp = next(part)
        assert torch.equal(tf[4:], tp) and torch.equal(lf[4:], lp)
        assert torch.equal(tf[:, 1:], lf[:, :-1])
    assert part.h2d_bytes_per_step == 4 * 9 * 8


def test_out_of_range_sample_is_an_error(corpus):
    prefix, _ = corpus
    data = D.IndexedDataset(prefix)
    ds = D.GPTTokenDataset(data, (0, 50), 8, 10, seed=0)
    native = D._native()
    out = np.empty((1, 9), dtype=np.int64)
    with pytest.raises(IndexError):
        native.gather_samples(data.raw, 2, data.pointers, data.sizes, ds.doc_idx, ds.sample_idx,
                              np.array([10 ** 9], dtype=np.int64), 8, out, 1)


def test_random_dataset_shapes():
    ds = D.RandomTokenDataset(100, 16, dataset_size=32)
    t, l = D.random_collate_fn([ds[0], ds[1]])
    assert t.shape == (2, 16) and l.shape == (2, 16)
