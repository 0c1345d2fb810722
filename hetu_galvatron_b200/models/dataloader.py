"""Random datasets of every family under the reference's names, for torch ``DataLoader`` based training loops.

The reference keeps one ``dataloader.py`` per model directory with a ``DataLoaderFor<Family>(args, device, dataset_size)``
dataset and a collate function (galvatron/models/llama_hf/dataloader.py:40-80, gpt_hf/dataloader.py:39-80,
bert_hf/dataloader.py:28-167, T5/dataloader.py:24-145, vit_hf/dataloader.py:24-58, swin/dataloader.py:24-58). Here they
live in one module and all collate functions return what ``GalvatronModel.forward_backward`` takes:
``(input, labels)`` or ``(input, labels, extras)`` with batch-major tensors and HuggingFace's names in the extras.

    ds = DataLoaderForBert(args, device)
    loader = distributed_dataloader(ds, args.global_train_batch_size, shuffle=True, collate_fn=random_collate_fn_bert, model=model)
    for batch in loader:
        loss = model.forward_backward(batch, it)

Samples are drawn once, on the host, from a seeded generator (``args.seed``, default 1234): every rank that builds the
dataset with the same arguments holds the same samples.
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import numpy as np
import torch
from torch.utils.data import Dataset

IGNORE = -100          # label value that the loss skips


def _seed(args) -> int:
    return int(getattr(args, "seed", 1234) or 1234)


# ---------------------------------------------------------------------------------------------------------- decoders
class _RandomSentences(Dataset):
    """Token sentences of random length (at least one token), zero padded to ``seq_length + 1`` so that inputs and
    next-token labels are two views of one row."""

    def __init__(self, args, device=None, dataset_size: int = 2560 * 16):
        self.vocab_size, self.seq_length, self.device = int(args.vocab_size), int(args.seq_length), device
        rng = np.random.RandomState(_seed(args))
        lengths = rng.randint(1, self.seq_length + 1, (dataset_size,))
        ids = rng.randint(0, self.vocab_size, (dataset_size, self.seq_length + 1))
        ids[np.arange(self.seq_length + 1)[None, :] >= lengths[:, None] + 1] = 0
        self.input_ids = torch.from_numpy(ids.astype(np.int64))
        self.lengths = torch.from_numpy(lengths.astype(np.int64))

    def __len__(self) -> int:
        return self.input_ids.shape[0]

    def __getitem__(self, i: int) -> torch.Tensor:
        row = self.input_ids[i]
        return row.to(self.device) if self.device is not None else row


class DataLoaderForLlama(_RandomSentences):
    pass


class DataLoaderForGPT(_RandomSentences):
    pass


def random_collate_fn(batch: Sequence[torch.Tensor]):
    """Rows of ``seq_length + 1`` tokens -> (input ids, next-token labels)."""
    t = torch.stack(list(batch), 0)
    return t[:, :-1].contiguous(), t[:, 1:].contiguous()


# ---------------------------------------------------------------------------------------------------------- BERT
class DataLoaderForBert(Dataset):
    """Sentence pairs ``[CLS] a [SEP] b [SEP] pad...`` with masked-language-model labels: 15 % of the ordinary tokens are
    chosen; of those 80 % become ``[MASK]``, 10 % another random token, 10 % stay; labels are the original ids at the chosen
    positions and ``-100`` elsewhere. Token types 0 / 1 mark the two sentences, the attention mask marks real tokens."""

    CLS, SEP, PAD, MASK = 101, 102, 0, 103

    def __init__(self, args, device=None, dataset_size: int = 64 * 16):
        self.vocab_size, self.seq_length, self.device = int(args.vocab_size), int(args.seq_length), device
        S = self.seq_length
        assert S >= 7 and self.vocab_size > 104, "need room for [CLS] a [SEP] b [SEP] and the special ids below the vocabulary"
        rng = np.random.RandomState(_seed(args))
        special = np.array([self.CLS, self.SEP, self.PAD, self.MASK])
        ordinary = np.setdiff1d(np.arange(self.vocab_size), special)
        shortest = min(2 * 10 + 3, S)                           # two sentences of ten tokens where the length allows
        total = rng.randint(shortest, S + 1, (dataset_size,))
        ids = np.full((dataset_size, S), self.PAD, dtype=np.int64)
        types = np.zeros((dataset_size, S), dtype=np.int64)
        mask = np.zeros((dataset_size, S), dtype=np.int64)
        for i, n in enumerate(total):
            body = n - 3
            shortest_sentence = min(10, body // 2)
            la = rng.randint(shortest_sentence, body - shortest_sentence + 1)
            lb = body - la
            row = np.concatenate([[self.CLS], rng.choice(ordinary, la), [self.SEP], rng.choice(ordinary, lb), [self.SEP]])
            ids[i, :n], mask[i, :n] = row, 1
            types[i, la + 2:n] = 1
        is_ordinary = (mask == 1) & ~np.isin(ids, special)
        chosen = is_ordinary & (rng.random_sample(ids.shape) < 0.15)
        labels = np.where(chosen, ids, IGNORE)
        fate = rng.random_sample(ids.shape)
        ids = np.where(chosen & (fate < 0.8), self.MASK, ids)
        swap = chosen & (fate >= 0.8) & (fate < 0.9)
        ids = np.where(swap, rng.choice(ordinary, ids.shape), ids)
        self.input_ids, self.attention_masks = torch.from_numpy(ids), torch.from_numpy(mask)
        self.token_type_ids, self.mlm_labels = torch.from_numpy(types), torch.from_numpy(labels)
        self.nsp_labels = torch.from_numpy(rng.randint(0, 2, (dataset_size,)).astype(np.int64))

    def __len__(self) -> int:
        return self.input_ids.shape[0]

    def __getitem__(self, i: int) -> Dict[str, torch.Tensor]:
        item = {"input_ids": self.input_ids[i], "attention_mask": self.attention_masks[i], "token_type_ids": self.token_type_ids[i],
                "mlm_labels": self.mlm_labels[i], "nsp_labels": self.nsp_labels[i:i + 1]}
        return {k: v.to(self.device) for k, v in item.items()} if self.device is not None else item


def random_collate_fn_bert(batch: Sequence[Dict[str, torch.Tensor]]):
    stack = lambda k: torch.stack([b[k] for b in batch], 0)
    return stack("input_ids"), stack("mlm_labels"), {"attention_mask": stack("attention_mask"), "token_type_ids": stack("token_type_ids")}


# ---------------------------------------------------------------------------------------------------------- T5
class DataLoaderForT5(Dataset):
    """Encoder and decoder sentences of random length, each padded to its own maximum (``encoder_seq_length`` /
    ``decoder_seq_length``, else ``seq_length``). The decoder input is the target shifted right behind the start token 0;
    labels are ``-100`` on padding."""

    def __init__(self, args, device=None, dataset_size: int = 2560 * 16):
        self.vocab_size, self.device = int(args.vocab_size), device
        self.encoder_seq_length = int(getattr(args, "encoder_seq_length", None) or args.seq_length)
        self.decoder_seq_length = int(getattr(args, "decoder_seq_length", None) or self.encoder_seq_length)
        se, sd = self.encoder_seq_length, self.decoder_seq_length
        rng = np.random.RandomState(_seed(args))
        enc_len, dec_len = rng.randint(1, se + 1, (dataset_size,)), rng.randint(1, sd + 1, (dataset_size,))
        enc = rng.randint(1, self.vocab_size, (dataset_size, se))
        tgt = rng.randint(1, self.vocab_size, (dataset_size, sd))
        self.enc_mask = torch.from_numpy((np.arange(se)[None, :] < enc_len[:, None]).astype(np.int64))
        self.dec_mask = torch.from_numpy((np.arange(sd)[None, :] < dec_len[:, None]).astype(np.int64))
        self.input_ids = torch.from_numpy(enc.astype(np.int64)) * self.enc_mask
        target = torch.from_numpy(tgt.astype(np.int64))
        self.labels = target.masked_fill(self.dec_mask == 0, IGNORE)
        self.decoder_input_ids = torch.cat([torch.zeros(dataset_size, 1, dtype=torch.int64), target[:, :-1]], 1) * self.dec_mask

    def __len__(self) -> int:
        return self.input_ids.shape[0]

    def __getitem__(self, i: int) -> Dict[str, torch.Tensor]:
        item = {"input_ids": self.input_ids[i], "attention_mask": self.enc_mask[i], "decoder_input_ids": self.decoder_input_ids[i],
                "decoder_attention_mask": self.dec_mask[i], "labels": self.labels[i]}
        return {k: v.to(self.device) for k, v in item.items()} if self.device is not None else item


def random_collate_fn_t5(batch: Sequence[Dict[str, torch.Tensor]]):
    stack = lambda k: torch.stack([b[k] for b in batch], 0)
    return stack("input_ids"), stack("labels"), {k: stack(k) for k in ("decoder_input_ids", "attention_mask", "decoder_attention_mask")}


# ---------------------------------------------------------------------------------------------------------- vision
class _RandomImages(Dataset):
    def __init__(self, args, device=None, dataset_size: int = 2560 * 16):
        self.device = device
        self.image_size, self.num_channels = int(args.image_size), int(getattr(args, "num_channels", 3) or 3)
        self.num_labels = int(getattr(args, "num_labels", None) or getattr(args, "num_classes", None) or 1000)
        self.dataset_size = dataset_size
        self.seed = _seed(args)
        self.labels = torch.from_numpy(np.random.RandomState(self.seed).randint(0, self.num_labels, (dataset_size,)).astype(np.int64))

    def __len__(self) -> int:
        return self.dataset_size

    def __getitem__(self, i: int):
        # pixels are drawn on demand from a per-sample seed: a dataset of thousands of images takes no memory
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + int(i))
        px = torch.randn(self.num_channels, self.image_size, self.image_size, generator=g)
        lb = self.labels[i]
        return (px.to(self.device), lb.to(self.device)) if self.device is not None else (px, lb)


class DataLoaderForViT(_RandomImages):
    pass


class DataLoaderForSwin(_RandomImages):
    pass


def vit_collate_fn(batch):
    """(pixels [C, H, W], label) pairs -> (pixel batch, labels)."""
    return torch.stack([b[0] for b in batch], 0), torch.stack([b[1] for b in batch], 0)


swin_collate_fn = vit_collate_fn

DATASETS = {"llama": (DataLoaderForLlama, random_collate_fn), "gpt": (DataLoaderForGPT, random_collate_fn),
            "bert": (DataLoaderForBert, random_collate_fn_bert), "t5": (DataLoaderForT5, random_collate_fn_t5),
            "vit": (DataLoaderForViT, vit_collate_fn), "swin": (DataLoaderForSwin, swin_collate_fn)}


def random_dataset(family: str, args, device=None, dataset_size: int = None):
    """(dataset, collate function) of a family by name (``llama_hf``, ``gpt_fa`` ... map to their base family)."""
    from .arguments import base_family

    cls, collate = DATASETS[base_family(family)]
    return (cls(args, device) if dataset_size is None else cls(args, device, dataset_size)), collate


def get_train_valid_test_data_iterators(args, cfg, model) -> List:
    """Token files named by ``--data-path`` as (train, validation, test) batch iterators of this rank (reference:
    ``get_train_valid_test_data_iterators`` of every decoder family, e.g. llama_hf/dataloader.py:107-131)."""
    from ..core.dataloader import build_token_iterator

    out = []
    for which in range(3):
        try:
            out.append(build_token_iterator(args, cfg, model, which=which))
        except ValueError:
            if which == 0:
                raise
            out.append(None)            # a split too small to hold a document (e.g. 1 per mille of a small corpus)
    return out
