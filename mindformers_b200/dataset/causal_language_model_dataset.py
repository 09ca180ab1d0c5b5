"""Datasets and loaders registered for the YAML ``train_dataset`` / ``train_dataset_task`` sections.

Reference: ``dataset/causal_language_model_dataset.py`` (:188-377: sharding by data-parallel rank, batching with
drop-remainder, EOD-reset maps, int32 cast), ``dataset/dataloader/blended_megatron_dataloader.py`` (:41-306: only
the first tensor-parallel rank of the first/last pipeline stage reads real data, others get fake samples),
``dataset/dataloader/*`` (common / SFT / indexed loaders), ``dataset/base_dataset.py`` (shard id / num shards).
Here everything is a ``torch.utils.data.DataLoader`` with a resumable sampler.
"""
from __future__ import annotations

import json
import os
from typing import Callable, Dict, Iterator, List, Optional

import numpy as np
import torch
from torch.utils.data import DataLoader, Dataset, Sampler

from ..parallel import parallel_state as ps
from ..tools.register import MindFormerModuleType, MindFormerRegister
from .gpt_dataset import BlendedMegatronDatasetBuilder, GPTDataset, GPTDatasetConfig, MockGPTDataset


class ResumableShardSampler(Sampler):
    """Deterministic shuffled shard of the index space with a fast-forward for resume (``set_init_step``)."""

    def __init__(self, size: int, num_shards: int = 1, shard_id: int = 0, shuffle: bool = False, seed: int = 0,
                 drop_last: bool = True):
        self.size, self.num_shards, self.shard_id = size, num_shards, shard_id
        self.shuffle, self.seed, self.drop_last = shuffle, seed, drop_last
        self.epoch, self.skip = 0, 0

    def set_epoch(self, epoch: int):
        self.epoch = epoch

    def set_skip(self, num_samples: int):
        self.skip = num_samples

    def __len__(self):
        return self.size // self.num_shards

    def __iter__(self) -> Iterator[int]:
        if self.shuffle:
            order = np.random.RandomState(self.seed + self.epoch).permutation(self.size)
        else:
            order = np.arange(self.size)
        per = self.size // self.num_shards
        mine = order[self.shard_id * per:(self.shard_id + 1) * per]
        start, self.skip = self.skip, 0
        return iter(mine[start:].tolist())


def collate(batch: List[Dict[str, torch.Tensor]]) -> Dict[str, torch.Tensor]:
    return {k: torch.stack([b[k] for b in batch]) for k in batch[0] if isinstance(batch[0][k], torch.Tensor)}


def data_shard_info():
    """(num_shards, shard_id) of this rank = its data-parallel coordinates."""
    return ps.get_data_parallel_world_size(), ps.get_data_parallel_rank()


class _TokenFileDataset(Dataset):
    """Pre-tokenised samples from a ``.npy`` / ``.jsonl`` file with an ``input_ids`` column."""

    def __init__(self, path: str, seq_length: int, column: str = "input_ids", pad_token_id: int = 0):
        self.seq_length, self.pad = seq_length, pad_token_id
        if path.endswith(".npy"):
            self.rows = np.load(path, mmap_mode="r")
        else:
            self.rows = []
            with open(path) as f:
                for line in f:
                    if line.strip():
                        self.rows.append(json.loads(line)[column])

    def __len__(self):
        return len(self.rows)

    def __getitem__(self, i):
        ids = np.asarray(self.rows[i], dtype=np.int64)[: self.seq_length + 1]
        if ids.shape[0] < self.seq_length + 1:
            ids = np.concatenate((ids, np.full(self.seq_length + 1 - ids.shape[0], self.pad, dtype=np.int64)))
        t = torch.from_numpy(ids.copy())
        return {"input_ids": t[:-1], "labels": t[1:], "loss_mask": (t[1:] != self.pad).float()}


@MindFormerRegister.register(MindFormerModuleType.DATASET_LOADER)
class BlendedMegatronDatasetDataLoader:
    """Factory for Megatron-format data (or synthetic data when ``mock: True`` / no ``data_path``)."""

    def __new__(cls, datasets_type: str = "GPTDataset", sizes=(1000, 0, 0), config: Optional[dict] = None,
                shuffle: bool = False, **kwargs):
        cfg = dict(config or {})
        data_path = cfg.pop("data_path", None)
        blend = None
        if data_path:
            prefixes, weights = [], []
            items = list(data_path)
            if len(items) > 1 and _is_number(items[0]):
                for w, p in zip(items[0::2], items[1::2]):
                    weights.append(float(w))
                    prefixes.append(p)
            else:
                prefixes = items
            blend = (prefixes, weights or None)
        known = {f.name for f in GPTDatasetConfig.__dataclass_fields__.values()}
        gcfg = GPTDatasetConfig(sequence_length=cfg.pop("seq_length", cfg.pop("sequence_length", 4096)), blend=blend,
                                **{k: v for k, v in cfg.items() if k in known})
        if blend is None:
            gcfg.mock = True
        # only the ranks that feed the model read files; the others get synthetic placeholders
        reader = ps.get_tensor_model_parallel_rank() == 0 and (ps.is_pipeline_first_stage(True) or ps.is_pipeline_last_stage(True))
        if not reader:
            gcfg.mock = True
        return BlendedMegatronDatasetBuilder(GPTDataset, list(sizes), gcfg).build()[0]


def _is_number(x) -> bool:
    try:
        float(x)
        return True
    except (TypeError, ValueError):
        return False


@MindFormerRegister.register(MindFormerModuleType.DATASET_LOADER)
class IndexedDataLoader:
    def __new__(cls, path_prefix: str, seq_length: int = 4096, num_samples: Optional[int] = None, seed: int = 1234, **kw):
        from .indexed_dataset import IndexedDataset
        indexed = IndexedDataset(path_prefix)
        gcfg = GPTDatasetConfig(sequence_length=seq_length, random_seed=seed)
        return GPTDataset(indexed, path_prefix, np.arange(len(indexed), dtype=np.int32), num_samples, "train", gcfg)


@MindFormerRegister.register(MindFormerModuleType.DATASET_LOADER)
class CommonDataLoader:
    """Pre-tokenised ``.jsonl`` / ``.npy`` files (the HF-datasets loader of the reference reduced to local files)."""

    def __new__(cls, path: str = None, dataset_dir: str = None, seq_length: int = 4096, input_columns=("input_ids",),
                pad_token_id: int = 0, **kw):
        return _TokenFileDataset(path or dataset_dir, seq_length, input_columns[0], pad_token_id)


@MindFormerRegister.register(MindFormerModuleType.DATASET_LOADER)
class MockDataLoader:
    def __new__(cls, seq_length: int = 4096, vocab_size: int = 32000, num_samples: int = 1 << 20, seed: int = 1234, **kw):
        return MockGPTDataset(num_samples, GPTDatasetConfig(sequence_length=seq_length, random_seed=seed,
                                                            vocab_size=vocab_size), vocab_size)


def build_dataset_loader(config: dict, default_args: Optional[dict] = None):
    return MindFormerRegister.get_instance_from_cfg(dict(config), MindFormerModuleType.DATASET_LOADER,
                                                    default_args=default_args)


@MindFormerRegister.register(MindFormerModuleType.DATASET)
class CausalLanguageModelDataset:
    """``CausalLanguageModelDataset(dataset_config)`` → batched iterator of dicts of tensors.

    Keys used from the configuration: ``data_loader`` (registry entry), ``batch_size``, ``drop_remainder``,
    ``shuffle``, ``seed``, ``num_parallel_workers``, ``input_columns``, ``pin_memory``.
    """

    def __new__(cls, dataset_config: Optional[dict] = None, **kwargs):
        cfg = dict(dataset_config or {})
        cfg.update(kwargs)
        loader_cfg = cfg.get("data_loader") or {"type": "MockDataLoader"}
        dataset = build_dataset_loader(loader_cfg) if isinstance(loader_cfg, dict) else loader_cfg
        shards, shard_id = data_shard_info()
        sampler = ResumableShardSampler(len(dataset), shards, shard_id, bool(cfg.get("shuffle", False)),
                                        int(cfg.get("seed", 0) or 0))
        loader = DataLoader(dataset, batch_size=int(cfg.get("batch_size", 1)), sampler=sampler,
                            drop_last=bool(cfg.get("drop_remainder", True)), collate_fn=collate,
                            num_workers=int(cfg.get("num_parallel_workers", 0) or 0),
                            pin_memory=bool(cfg.get("pin_memory", torch.cuda.is_available())))
        loader.shard_sampler = sampler
        loader.set_init_step = lambda steps, bs=int(cfg.get("batch_size", 1)): sampler.set_skip(steps * bs)
        return loader


@MindFormerRegister.register(MindFormerModuleType.DATASET)
class KeyWordGenDataset(CausalLanguageModelDataset):
    """Prompt/answer generation data; batches carry ``input_ids``/``labels`` like the causal dataset."""


@MindFormerRegister.register(MindFormerModuleType.DATASET)
class MultiTurnDataset(CausalLanguageModelDataset):
    """Multi-turn chat data with per-turn loss masks."""


@MindFormerRegister.register(MindFormerModuleType.DATASET)
class GeneralDataset(CausalLanguageModelDataset):
    """Any map-style dataset object passed as ``data_loader``."""


def build_dataset(config: Optional[dict] = None, default_args: Optional[dict] = None, **kwargs):
    """``config = {"type": "CausalLanguageModelDataset", "dataset_config": {...}}`` (the YAML ``*_dataset_task``)."""
    if config is None:
        return None
    cfg = dict(config)
    cfg.update(kwargs)
    return MindFormerRegister.get_instance_from_cfg(cfg, MindFormerModuleType.DATASET, default_args=default_args)
