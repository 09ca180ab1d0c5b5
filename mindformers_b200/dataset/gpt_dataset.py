"""GPT pre-training datasets over indexed token files, weighted blends, and synthetic data.

Reference: ``dataset/blended_datasets/gpt_dataset.py`` (``GPTDataset`` index building and caching :313-516,
``__getitem__`` :170-239, EOD-reset masks :639-712, compressed EOD mask :612-636, ``MockGPTDataset`` :740),
``blended_dataset.py``, ``blended_megatron_dataset_builder.py``. A sample is
``(tokens[:-1], labels = tokens[1:], loss_mask, position_ids[, actual_seq_len])``: the label shift happens here,
not in the model.
"""
from __future__ import annotations

import enum
import hashlib
import json
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import helpers
from .indexed_dataset import IndexedDataset


@dataclass
class GPTDatasetConfig:
    """Settings of the Megatron-style GPT dataset: sequence length, seed, split, blend, end-of-document handling
    (``reset_position_ids``, ``reset_attention_mask``, ``eod_mask_loss``, ``create_compressed_eod_mask``), cache
    directory."""

    sequence_length: int
    random_seed: int = 1234
    blend: Optional[Tuple[List[str], Optional[List[float]]]] = None
    split: str = "1,0,0"
    path_to_cache: Optional[str] = None
    reset_position_ids: bool = False
    reset_attention_mask: bool = False
    eod_mask_loss: bool = False
    create_attention_mask: bool = False
    create_compressed_eod_mask: bool = False
    eod_pad_length: int = 128
    eod: int = 0
    pad: int = -1
    drop_last_partial_sequence: bool = True
    add_extra_token_to_sequence: bool = True
    mock: bool = False
    vocab_size: Optional[int] = None


def parse_split(split: str) -> List[float]:
    parts = [float(x) for x in str(split).replace("/", ",").split(",")]
    parts += [0.0] * (3 - len(parts))
    s = sum(parts)
    if s <= 0:
        raise ValueError(f"split {split!r} has no positive entry")
    return [p / s for p in parts[:3]]


class Split(enum.Enum):
    train = 0
    valid = 1
    test = 2


def normalize(weights: Sequence[float]) -> List[float]:
    """Weights divided by their sum (float64)."""
    w = np.asarray(weights, dtype=np.float64)
    return (w / w.sum()).tolist()


def parse_and_normalize_split(split: str) -> List[float]:
    """``"99,1,0"`` / ``"99/1"`` → three fractions that sum to 1."""
    return parse_split(split)


def convert_split_vector_to_split_matrix(vector_a: Sequence[float], vector_b: Optional[Sequence[float]] = None):
    """Fractions → ``[(begin, end) or None]`` bookends on [0, 1] per split; with a second vector, the overlap of the two
    layouts per split (used to carve a retrieval corpus from the same documents)."""
    def bookends(v):
        edges = np.concatenate([[0.0], np.cumsum(np.asarray(v, dtype=np.float64))])
        return [(float(edges[i]), float(edges[i + 1])) if edges[i + 1] > edges[i] else None for i in range(len(v))]

    a = bookends(vector_a)
    if vector_b is None:
        return a
    out = []
    for x, y in zip(a, bookends(vector_b)):
        if x is None or y is None:
            out.append(None)
            continue
        lo, hi = max(x[0], y[0]), min(x[1], y[1])
        out.append((lo, hi) if hi > lo else None)
    return out


def get_blend_from_list(blend: Optional[Sequence[str]]):
    """``["30", "a_prefix", "70", "b_prefix"]`` → ``(["a_prefix", "b_prefix"], [30.0, 70.0])``; a plain list of prefixes →
    ``(prefixes, None)``; None → None."""
    if blend is None:
        return None
    items = [str(b).strip() for b in blend]
    if len(items) % 2 == 0:
        try:
            weights = [float(w) for w in items[0::2]]
            return items[1::2], weights
        except ValueError:
            pass
    return items, None


BlendedMegatronDatasetConfig = GPTDatasetConfig


class GPTDataset(torch.utils.data.Dataset):
    """Fixed-length samples cut from a shuffled concatenation of documents."""

    def __init__(self, indexed: IndexedDataset, dataset_path: Optional[str], indexed_indices: np.ndarray,
                 num_samples: Optional[int], index_split: str, config: GPTDatasetConfig):
        self.dataset, self.dataset_path = indexed, dataset_path
        self.indices = np.asarray(indexed_indices, dtype=np.int32)
        self.num_samples, self.index_split, self.config = num_samples, index_split, config
        self.document_index, self.sample_index, self.shuffle_index = self._build_indices()

    # ---- index construction ------------------------------------------------------------------------
    def _description(self) -> str:
        c = self.config
        return json.dumps({"class": type(self).__name__, "path": self.dataset_path, "num_samples": self.num_samples,
                           "split": self.index_split, "seed": c.random_seed, "seq": c.sequence_length,
                           "indices": [int(self.indices[0]), int(self.indices[-1]), len(self.indices)] if len(self.indices) else [],
                           "drop_last": c.drop_last_partial_sequence, "extra": c.add_extra_token_to_sequence}, indent=1)

    def _build_indices(self):
        c = self.config
        desc = self._description()
        digest = hashlib.md5(desc.encode()).hexdigest()
        cache = c.path_to_cache
        names = None
        if cache:
            os.makedirs(cache, exist_ok=True)
            base = os.path.join(cache, f"{digest}-{type(self).__name__}-{self.index_split}")
            names = {k: f"{base}-{k}_index.npy" for k in ("document", "sample", "shuffle")}
            if all(os.path.exists(p) for p in names.values()):
                return tuple(np.load(names[k], allow_pickle=False, mmap_mode="r") for k in ("document", "sample", "shuffle"))
        sizes = np.asarray(self.dataset.sequence_lengths, dtype=np.int32)
        extra = 1 if c.add_extra_token_to_sequence else 0
        tokens_per_epoch = int(sizes[self.indices].sum())
        if tokens_per_epoch <= 1:
            raise ValueError("dataset split is empty")
        seq = c.sequence_length
        if self.num_samples is None:
            num_epochs = 1
        else:
            num_epochs = 1
            while (num_epochs * tokens_per_epoch - extra) // seq < self.num_samples:
                num_epochs += 1
        rng = np.random.RandomState(c.random_seed)
        # the last epoch is shuffled separately when only a small part of it is needed, so that early
        # samples are not dominated by a partial epoch (same rule as Megatron)
        separate_last = False
        if num_epochs > 1 and self.num_samples is not None:
            per_epoch = (tokens_per_epoch - extra) // seq
            from_last = self.num_samples - ((num_epochs - 1) * tokens_per_epoch - extra) // seq
            separate_last = from_last < int(0.80 * per_epoch)
        document_index = self._document_index(num_epochs, rng, separate_last)
        sample_index = helpers.build_sample_idx(sizes, document_index, seq, num_epochs, tokens_per_epoch,
                                                c.drop_last_partial_sequence, extra)
        n = sample_index.shape[0] - 1
        if separate_last:
            head = ((num_epochs - 1) * tokens_per_epoch - extra) // seq
            shuffle_index = np.concatenate((rng.permutation(head), head + rng.permutation(n - head))).astype(np.uint32)
        else:
            shuffle_index = rng.permutation(n).astype(np.uint32)
        if names:
            with open(names["document"].replace("-document_index.npy", "-description.txt"), "w") as f:
                f.write(desc)
            np.save(names["document"], document_index, allow_pickle=False)
            np.save(names["sample"], sample_index, allow_pickle=False)
            np.save(names["shuffle"], shuffle_index, allow_pickle=False)
        return document_index, sample_index, shuffle_index

    def _document_index(self, num_epochs: int, rng, separate_last: bool) -> np.ndarray:
        if not separate_last or num_epochs == 1:
            doc = np.tile(self.indices, num_epochs).astype(np.int32)
            rng.shuffle(doc)
            return doc
        first = np.tile(self.indices, num_epochs - 1).astype(np.int32)
        rng.shuffle(first)
        last = self.indices.copy().astype(np.int32)
        rng.shuffle(last)
        return np.concatenate((first, last))

    # ---- access ------------------------------------------------------------------------------------
    def __len__(self):
        return self.sample_index.shape[0] - 1

    def _tokens(self, idx: int) -> np.ndarray:
        idx = int(self.shuffle_index[idx])
        d0, o0 = self.sample_index[idx]
        d1, o1 = self.sample_index[idx + 1]
        extra = 1 if self.config.add_extra_token_to_sequence else 0
        if d0 == d1:
            return np.asarray(self.dataset.get(int(self.document_index[d0]), int(o0), int(o1 - o0 + extra)), dtype=np.int64)
        parts = []
        for d in range(int(d0), int(d1) + 1):
            doc = int(self.document_index[d])
            off = int(o0) if d == d0 else 0
            length = int(o1) + extra if d == d1 else None
            parts.append(self.dataset.get(doc, off, length))
        return np.concatenate(parts).astype(np.int64)

    def __getitem__(self, idx: int) -> Dict[str, torch.Tensor]:
        c = self.config
        text = self._tokens(idx % len(self))
        need = c.sequence_length + (1 if c.add_extra_token_to_sequence else 0)
        if text.shape[0] < need:
            text = np.concatenate((text, np.full(need - text.shape[0], c.pad if c.pad >= 0 else c.eod, dtype=np.int64)))
        tokens, labels = text[:-1], text[1:]
        return build_sample(torch.from_numpy(tokens.copy()), torch.from_numpy(labels.copy()), c)


def build_sample(tokens: torch.Tensor, labels: torch.Tensor, c: GPTDatasetConfig) -> Dict[str, torch.Tensor]:
    S = tokens.shape[0]
    loss_mask = torch.ones(S, dtype=torch.float32)
    if c.eod_mask_loss:
        loss_mask[tokens == c.eod] = 0.0
    if c.pad >= 0:
        loss_mask[labels == c.pad] = 0.0
    position_ids = torch.arange(S, dtype=torch.int64)
    out = {"input_ids": tokens, "labels": labels, "loss_mask": loss_mask, "position_ids": position_ids}
    eod_pos = (tokens == c.eod).nonzero().flatten()
    if c.reset_position_ids and eod_pos.numel():
        prev = 0
        for e in eod_pos.tolist():
            position_ids[e + 1:] -= (e + 1 - prev)
            prev = e + 1
    if c.create_compressed_eod_mask:
        # cumulative sequence lengths of the packed documents, padded to a fixed length (TND layout)
        ends = (eod_pos + 1).tolist()
        if not ends or ends[-1] != S:
            ends.append(S)
        ends = ends[: c.eod_pad_length]
        ends[-1] = S
        asl = torch.full((c.eod_pad_length,), S, dtype=torch.int32)
        asl[: len(ends)] = torch.tensor(ends, dtype=torch.int32)
        out["actual_seq_len"] = asl
    elif c.create_attention_mask:
        mask = torch.tril(torch.ones(S, S, dtype=torch.bool))
        if c.reset_attention_mask:
            for e in eod_pos.tolist():
                mask[e + 1:, : e + 1] = False
        out["attention_mask"] = ~mask
    return out


class MockGPTDataset(torch.utils.data.Dataset):
    """Synthetic uniform token ids; deterministic per index (used by benchmarks and non-reader ranks)."""

    def __init__(self, num_samples: int, config: GPTDatasetConfig, vocab_size: Optional[int] = None):
        self.num_samples, self.config = num_samples, config
        self.vocab_size = vocab_size or config.vocab_size or 32000

    def __len__(self):
        return self.num_samples

    def __getitem__(self, idx):
        g = torch.Generator().manual_seed(self.config.random_seed * 1000003 + int(idx))
        text = torch.randint(0, self.vocab_size, (self.config.sequence_length + 1,), generator=g, dtype=torch.int64)
        return build_sample(text[:-1].clone(), text[1:].clone(), self.config)


class BlendedDataset(torch.utils.data.Dataset):
    """Weighted interleave of several datasets (greedy error-minimising order from the native helper)."""

    def __init__(self, datasets: Sequence[torch.utils.data.Dataset], weights: Optional[Sequence[float]],
                 size: Optional[int]):
        self.datasets = list(datasets)
        n = len(self.datasets)
        if weights is None:
            sizes = [len(d) for d in self.datasets]
            total = sum(sizes)
            self.dataset_index = np.zeros(total, dtype=np.int16)
            self.dataset_sample_index = np.zeros(total, dtype=np.int64)
            helpers.build_exhaustive_blending_indices(self.dataset_index, self.dataset_sample_index, sizes, n)
        else:
            w = np.asarray(weights, dtype=np.float64)
            w = w / w.sum()
            size = int(size if size is not None else sum(len(d) for d in self.datasets))
            self.dataset_index = np.zeros(size, dtype=np.int16)
            self.dataset_sample_index = np.zeros(size, dtype=np.int64)
            helpers.build_blending_indices(self.dataset_index, self.dataset_sample_index, w, n, size)

    def __len__(self):
        return self.dataset_index.shape[0]

    def __getitem__(self, idx):
        d = int(self.dataset_index[idx])
        s = int(self.dataset_sample_index[idx])
        item = self.datasets[d][s % len(self.datasets[d])]
        return dict(item, dataset_id=torch.tensor(d))


class BlendedMegatronDatasetBuilder:
    """Build (train, valid, test) datasets from ``config.blend`` = (prefixes, weights) and ``config.split``."""

    def __init__(self, cls, sizes: Sequence[Optional[int]], config: GPTDatasetConfig):
        self.cls, self.sizes, self.config = cls, list(sizes), config

    def build(self) -> List[Optional[torch.utils.data.Dataset]]:
        c = self.config
        if c.mock or not c.blend:
            return [MockGPTDataset(n, c) if n else None for n in self.sizes]
        prefixes, weights = c.blend
        fractions = parse_split(c.split)
        per_split: List[List] = [[], [], []]
        for prefix in prefixes:
            indexed = IndexedDataset(prefix)
            n_docs = len(indexed.document_indices) - 1
            bounds = [0]
            for f in fractions:
                bounds.append(bounds[-1] + int(round(f * n_docs)))
            bounds[-1] = n_docs
            for i, name in enumerate(("train", "valid", "test")):
                lo, hi = bounds[i], bounds[i + 1]
                if hi <= lo or not self.sizes[i]:
                    per_split[i].append(None)
                    continue
                seq_lo, seq_hi = int(indexed.document_indices[lo]), int(indexed.document_indices[hi])
                share = self.sizes[i]
                if weights:
                    w = weights[prefixes.index(prefix)] / sum(weights)
                    share = int(np.ceil(self.sizes[i] * w * 1.005))
                per_split[i].append(self.cls(indexed, prefix, np.arange(seq_lo, seq_hi, dtype=np.int32), share, name, c))
        out = []
        for i in range(3):
            parts = [d for d in per_split[i] if d is not None]
            if not parts:
                out.append(None)
            elif len(parts) == 1:
                out.append(parts[0])
            else:
                out.append(BlendedDataset(parts, weights, self.sizes[i]))
        return out
