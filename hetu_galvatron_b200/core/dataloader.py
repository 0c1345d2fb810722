"""Token datasets: Megatron-style indexed files (``<prefix>.idx`` + ``<prefix>.bin``), epoch shuffling, blending, and
the per-rank batch iterator of the training loop.

The reference reaches Megatron's ``GPTDataset`` / ``BlendedMegatronDatasetBuilder`` through
``build_train_valid_test_data_iterators`` (galvatron/core/runtime/dataloader.py:1-10,
galvatron/models/llama_hf/dataloader.py:107-164) and broadcasts every batch from the TP source rank. Here every rank
builds the same index deterministically from the seed, reads ONLY its data-parallel slice of each global batch, and
assembles it with the native ``data_index.gather_samples`` straight into a pinned host buffer followed by one
asynchronous H2D copy — no broadcast, no worker processes.

On-disk format (Megatron ``MMapIndexedDataset``): ``.idx`` = magic ``MMIDIDX\\0\\0`` | u64 version (1) | u8 dtype code |
u64 sequence count | u64 document count | int32 sizes[seq] | int64 byte pointers[seq] | int64 document boundaries[doc];
``.bin`` = the tokens back to back.
"""
from __future__ import annotations

import struct
from typing import Iterator, List, Sequence, Tuple

import numpy as np
import torch

_MAGIC = b"MMIDIDX\x00\x00"
_DTYPES = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float64, 7: np.float32, 8: np.uint16}
_CODES = {np.dtype(v).name: k for k, v in _DTYPES.items()}


def _native():
    from .._build import load_pybind
    return load_pybind("data_index")


def write_indexed_dataset(prefix: str, documents: Sequence[Sequence[int]], dtype=np.uint16) -> None:
    """Write ``documents`` (token id lists) as ``prefix.idx`` / ``prefix.bin``."""
    dtype = np.dtype(dtype)
    sizes = np.array([len(d) for d in documents], dtype=np.int32)
    pointers = np.zeros(len(documents), dtype=np.int64)
    if len(documents) > 1:
        pointers[1:] = np.cumsum(sizes[:-1].astype(np.int64)) * dtype.itemsize
    with open(prefix + ".bin", "wb") as fb:
        for d in documents:
            fb.write(np.asarray(d, dtype=dtype).tobytes())
    with open(prefix + ".idx", "wb") as fi:
        fi.write(_MAGIC)
        fi.write(struct.pack("<Q", 1))
        fi.write(struct.pack("<B", _CODES[dtype.name]))
        fi.write(struct.pack("<Q", len(sizes)))
        fi.write(struct.pack("<Q", len(sizes) + 1))
        fi.write(sizes.tobytes())
        fi.write(pointers.tobytes())
        fi.write(np.arange(len(sizes) + 1, dtype=np.int64).tobytes())


class IndexedDataset:
    """Read-only memory-mapped view of one ``.idx`` / ``.bin`` pair."""

    def __init__(self, prefix: str):
        with open(prefix + ".idx", "rb") as f:
            if f.read(9) != _MAGIC:
                raise ValueError("%s.idx is not an indexed-dataset index file" % prefix)
            (version,) = struct.unpack("<Q", f.read(8))
            if version != 1:
                raise ValueError("unsupported index version %d" % version)
            (code,) = struct.unpack("<B", f.read(1))
            (n_seq,) = struct.unpack("<Q", f.read(8))
            (n_doc,) = struct.unpack("<Q", f.read(8))
            header = f.tell()
        self.dtype = np.dtype(_DTYPES[code])
        if self.dtype.itemsize not in (2, 4):
            raise ValueError("token width %d is not supported (2 or 4 bytes)" % self.dtype.itemsize)
        idx = np.memmap(prefix + ".idx", mode="r", order="C")
        self.sizes = np.frombuffer(idx, dtype=np.int32, count=n_seq, offset=header)
        self.pointers = np.frombuffer(idx, dtype=np.int64, count=n_seq, offset=header + self.sizes.nbytes)
        self.doc_bounds = np.frombuffer(idx, dtype=np.int64, count=n_doc, offset=header + self.sizes.nbytes + self.pointers.nbytes)
        self.raw = np.memmap(prefix + ".bin", mode="r", dtype=np.uint8, order="C")

    def __len__(self) -> int:
        return len(self.sizes)

    def document(self, i: int) -> np.ndarray:
        lo = int(self.pointers[i])
        return np.frombuffer(self.raw, dtype=self.dtype, count=int(self.sizes[i]), offset=lo)


def split_ranges(n_docs: int, split: str) -> List[Tuple[int, int]]:
    """``"969,30,1"`` -> document ranges of train / valid / test (Megatron's ``--split``)."""
    parts = [float(x) for x in split.replace("/", ",").split(",") if x != ""]
    parts = (parts + [0.0, 0.0, 0.0])[:3]
    total = sum(parts) or 1.0
    bounds, acc = [0], 0.0
    for p in parts:
        acc += p / total
        bounds.append(int(round(acc * n_docs)))
    bounds[-1] = n_docs
    return [(bounds[i], bounds[i + 1]) for i in range(3)]


class GPTTokenDataset:
    """Fixed-length samples (``seq_length + 1`` tokens) cut from the shuffled concatenation of the documents of one
    split, for as many epochs as ``num_samples`` needs (Megatron ``GPTDataset`` semantics: per-epoch document
    shuffle, sample index over the stream, shuffled sample order)."""

    def __init__(self, data: IndexedDataset, doc_range: Tuple[int, int], seq_length: int, num_samples: int, seed: int):
        self.data, self.seq_length = data, seq_length
        docs = np.arange(doc_range[0], doc_range[1], dtype=np.int32)
        if len(docs) == 0:
            raise ValueError("empty document range")
        tokens_per_epoch = int(data.sizes[docs].astype(np.int64).sum())
        epochs = 1
        while (epochs * tokens_per_epoch - 1) // seq_length < num_samples:
            epochs += 1
        rng = np.random.RandomState(seed)
        self.doc_idx = np.concatenate([rng.permutation(docs) for _ in range(epochs)]).astype(np.int32)
        self.sample_idx = np.ascontiguousarray(
            _native().build_sample_idx(np.ascontiguousarray(data.sizes), self.doc_idx, seq_length, epochs, tokens_per_epoch)
        ).astype(np.int64)
        self.shuffle_idx = rng.permutation(len(self.sample_idx) - 1).astype(np.int64)
        self.num_samples = len(self.shuffle_idx)

    def __len__(self) -> int:
        return self.num_samples

    def gather(self, picks: np.ndarray, out: np.ndarray, threads: int = 8) -> None:
        """Fill ``out[len(picks), seq_length + 1]`` (int64) with the samples ``picks`` (positions in shuffled order)."""
        real = self.shuffle_idx[np.asarray(picks, dtype=np.int64) % self.num_samples]
        _native().gather_samples(self.data.raw, self.data.dtype.itemsize, self.data.pointers, self.data.sizes, self.doc_idx,
                                 self.sample_idx, np.ascontiguousarray(real), self.seq_length, out, threads)

    def __getitem__(self, i: int) -> np.ndarray:
        out = np.empty((1, self.seq_length + 1), dtype=np.int64)
        self.gather(np.array([i]), out, 1)
        return out[0]


class BlendedDataset:
    """Weighted interleave of several datasets (Megatron ``BlendedDataset``)."""

    def __init__(self, datasets: Sequence[GPTTokenDataset], weights: Sequence[float], size: int):
        w = np.asarray(weights, dtype=np.float64)
        self.datasets = list(datasets)
        self.which, self.index = _native().build_blending_indices(w / w.sum(), size)
        self.seq_length = datasets[0].seq_length
        self.num_samples = size

    def __len__(self) -> int:
        return self.num_samples

    def gather(self, picks: np.ndarray, out: np.ndarray, threads: int = 8) -> None:
        picks = np.asarray(picks, dtype=np.int64) % self.num_samples
        which, index = self.which[picks], self.index[picks]
        for d, ds in enumerate(self.datasets):
            rows = np.nonzero(which == d)[0]
            if len(rows):
                tmp = np.empty((len(rows), self.seq_length + 1), dtype=np.int64)
                ds.gather(index[rows], tmp, threads)
                out[rows] = tmp


def parse_data_path(data_path) -> Tuple[List[str], List[float]]:
    """``["p"]`` or ``["0.3", "p1", "0.7", "p2"]`` -> prefixes, weights."""
    items = list(data_path) if isinstance(data_path, (list, tuple)) else str(data_path).split()
    if len(items) == 1:
        return [items[0]], [1.0]
    if len(items) % 2:
        raise ValueError("--data-path takes one prefix or weight/prefix pairs")
    return [items[i + 1] for i in range(0, len(items), 2)], [float(items[i]) for i in range(0, len(items), 2)]


def build_dataset(data_path, seq_length: int, num_samples: int, seed: int, split: str = "969,30,1", which: int = 0):
    prefixes, weights = parse_data_path(data_path)
    parts = []
    for p, w in zip(prefixes, weights):
        data = IndexedDataset(p)
        rng = split_ranges(len(data), split)[which]
        share = num_samples if len(prefixes) == 1 else int(np.ceil(num_samples * w / sum(weights) * 1.005)) + 1
        parts.append(GPTTokenDataset(data, rng, seq_length, share, seed))
    return parts[0] if len(parts) == 1 else BlendedDataset(parts, weights, num_samples)


class TokenBatchIterator:
    """Yields ``(tokens [b_local, s], labels [b_local, s])`` on ``device`` for this rank's slice ``[lo, hi)`` of every
    global batch. Two pinned staging buffers alternate so the H2D copy of batch i overlaps the host gather of i+1."""

    def __init__(self, dataset, global_batch: int, lo: int, hi: int, device, start_iter: int = 0, threads: int = 8):
        self.ds, self.gb, self.lo, self.hi, self.device = dataset, global_batch, lo, hi, device
        self.iter = start_iter
        self.threads = threads
        n, span = hi - lo, dataset.seq_length + 1
        pin = torch.cuda.is_available() and torch.device(device).type == "cuda"
        self._host = [torch.empty(n, span, dtype=torch.int64, pin_memory=pin) for _ in range(2)]
        self._events = [None, None]
        self.h2d_bytes_per_step = n * span * 8

    def __iter__(self) -> Iterator:
        return self

    def __next__(self):
        k = self.iter & 1
        if self._events[k] is not None:
            self._events[k].synchronize()
        first = self.iter * self.gb + self.lo
        picks = np.arange(first, first + (self.hi - self.lo), dtype=np.int64)
        self.ds.gather(picks, self._host[k].numpy(), self.threads)
        dev = self._host[k].to(self.device, non_blocking=True)
        if dev.is_cuda:
            ev = torch.cuda.Event()
            ev.record()
            self._events[k] = ev
        self.iter += 1
        return dev[:, :-1].contiguous(), dev[:, 1:].contiguous()


def build_token_iterator(args, cfg, model, which: int = 0) -> TokenBatchIterator:
    """The training loop's data iterator from ``--data-path`` / ``--split`` (reference: llama_hf/dataloader.py:107-131)."""
    gb = args.global_train_batch_size
    iters = getattr(args, "train_iters", None) or 25
    ds = build_dataset(args.data_path, cfg.seq_length, gb * iters, getattr(args, "seed", 1234), getattr(args, "split", "969,30,1"), which)
    lo, hi = model.batch_slice()
    start = args.load_iteration if getattr(args, "distributed_checkpoint", False) and getattr(args, "load", None) else 0
    return TokenBatchIterator(ds, gb, lo, hi, model.device, start_iter=start)


class RandomTokenDataset(torch.utils.data.Dataset):
    """Random token sentences of random length, zero padded (reference: llama_hf/dataloader.py:52-80
    ``DataLoaderForLlama``); used by ``train_dist_random`` style runs that want a torch ``DataLoader``."""

    def __init__(self, vocab_size: int, seq_length: int, dataset_size: int = 2560 * 16, seed: int = 1234):
        rng = np.random.RandomState(seed)
        lengths = rng.randint(1, seq_length + 1, (dataset_size,))
        ids = rng.randint(0, vocab_size, (dataset_size, seq_length + 1))
        ids[np.arange(seq_length + 1)[None, :] >= lengths[:, None]] = 0
        self.input_ids = torch.from_numpy(ids.astype(np.int64))

    def __len__(self) -> int:
        return self.input_ids.shape[0]

    def __getitem__(self, i: int) -> torch.Tensor:
        return self.input_ids[i]


def random_collate_fn(batch):
    t = torch.stack(batch, 0)
    return t[:, :-1].contiguous(), t[:, 1:].contiguous()
