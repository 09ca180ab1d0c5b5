"""``build_sampler``: dataset samplers from configuration (reference ``dataset/sampler/build_sampler.py:23-67``, which
registers MindSpore's built-in samplers under ``MindFormerModuleType.DATASET_SAMPLER``). The same names map onto
``torch.utils.data`` samplers; ``DistributedSampler`` takes MindSpore's ``num_shards`` / ``shard_id`` arguments, and
``PKSampler`` (``num_val`` samples of every class, classes in order or shuffled) is implemented here because torch has
no counterpart."""
from __future__ import annotations

import random
from typing import Dict, Iterator, List, Optional, Sequence

import torch
from torch.utils.data import Sampler
from torch.utils.data import (RandomSampler as _TorchRandom, SequentialSampler as _TorchSequential,
                              SubsetRandomSampler as _TorchSubsetRandom, WeightedRandomSampler as _TorchWeighted)

from ..tools.register import MindFormerModuleType, MindFormerRegister


class _Sized:
    """Stands in for the dataset where only its length is known (MindSpore samplers take ``num_samples``, not a dataset)."""

    def __init__(self, n: int):
        self.n = int(n)

    def __len__(self):
        return self.n


@MindFormerRegister.register(MindFormerModuleType.DATASET_SAMPLER)
class SequentialSampler(Sampler):
    def __init__(self, data_source=None, start_index: int = 0, num_samples: Optional[int] = None, dataset_size: Optional[int] = None):
        self.size = len(data_source) if data_source is not None else int(dataset_size or (start_index + (num_samples or 0)))
        self.start, self.num = int(start_index or 0), num_samples

    def __iter__(self) -> Iterator[int]:
        end = self.size if self.num is None else min(self.size, self.start + self.num)
        return iter(range(self.start, end))

    def __len__(self):
        return max(0, (self.size if self.num is None else min(self.size, self.start + self.num)) - self.start)


@MindFormerRegister.register(MindFormerModuleType.DATASET_SAMPLER)
class RandomSampler(_TorchRandom):
    def __init__(self, data_source=None, replacement: bool = False, num_samples: Optional[int] = None,
                 dataset_size: Optional[int] = None, seed: Optional[int] = None):
        src = data_source if data_source is not None else _Sized(dataset_size or num_samples or 0)
        gen = torch.Generator().manual_seed(int(seed)) if seed is not None else None
        super().__init__(src, replacement=replacement, num_samples=num_samples if (replacement or num_samples) else None,
                         generator=gen)


@MindFormerRegister.register(MindFormerModuleType.DATASET_SAMPLER)
class SubsetRandomSampler(_TorchSubsetRandom):
    def __init__(self, indices: Sequence[int], num_samples: Optional[int] = None, seed: Optional[int] = None):
        gen = torch.Generator().manual_seed(int(seed)) if seed is not None else None
        super().__init__(list(indices), generator=gen)
        self.num = num_samples

    def __iter__(self):
        it = super().__iter__()
        return it if self.num is None else (i for _, i in zip(range(self.num), it))

    def __len__(self):
        return len(self.indices) if self.num is None else min(self.num, len(self.indices))


@MindFormerRegister.register(MindFormerModuleType.DATASET_SAMPLER)
class SubsetSampler(Sampler):
    """The given indices in their order."""

    def __init__(self, indices: Sequence[int], num_samples: Optional[int] = None):
        self.indices = list(indices)[: num_samples if num_samples is not None else None]

    def __iter__(self):
        return iter(self.indices)

    def __len__(self):
        return len(self.indices)


@MindFormerRegister.register(MindFormerModuleType.DATASET_SAMPLER)
class WeightedRandomSampler(_TorchWeighted):
    def __init__(self, weights: Sequence[float], num_samples: Optional[int] = None, replacement: bool = True,
                 seed: Optional[int] = None):
        gen = torch.Generator().manual_seed(int(seed)) if seed is not None else None
        super().__init__(list(weights), num_samples or len(weights), replacement=replacement, generator=gen)


@MindFormerRegister.register(MindFormerModuleType.DATASET_SAMPLER)
class DistributedSampler(Sampler):
    """Every ``num_shards``-th sample starting at ``shard_id`` (+ ``offset``), after an optional seeded shuffle that is
    the same on all shards; the tail is padded by wrapping around so that every shard has the same length."""

    def __init__(self, num_shards: int, shard_id: int, shuffle: bool = True, num_samples: Optional[int] = None,
                 offset: int = -1, dataset_size: Optional[int] = None, data_source=None, seed: int = 0):
        if not 0 <= shard_id < num_shards:
            raise ValueError(f"shard_id {shard_id} must be in [0, {num_shards})")
        self.size = len(data_source) if data_source is not None else int(dataset_size or 0)
        self.num_shards, self.shard_id, self.shuffle, self.num, self.seed = num_shards, shard_id, shuffle, num_samples, seed
        self.offset = max(0, offset)
        self.epoch = 0

    def set_epoch(self, epoch: int):
        self.epoch = int(epoch)

    def _order(self) -> List[int]:
        idx = list(range(self.size))
        if self.shuffle:
            random.Random(self.seed + self.epoch).shuffle(idx)
        per = -(-self.size // self.num_shards)
        idx += idx[: per * self.num_shards - len(idx)]
        mine = idx[(self.shard_id + self.offset) % self.num_shards::self.num_shards]
        return mine if self.num is None else mine[: self.num]

    def __iter__(self):
        return iter(self._order())

    def __len__(self):
        per = -(-self.size // self.num_shards)
        return per if self.num is None else min(per, self.num)


@MindFormerRegister.register(MindFormerModuleType.DATASET_SAMPLER)
class PKSampler(Sampler):
    """``num_val`` samples of each class per pass (``labels[i]`` is the class of sample ``i``)."""

    def __init__(self, num_val: int, labels: Sequence[int], num_class: Optional[int] = None, shuffle: bool = False,
                 class_column: str = "label", num_samples: Optional[int] = None, seed: int = 0):
        self.num_val, self.shuffle, self.num, self.seed = int(num_val), shuffle, num_samples, seed
        by_class: Dict[int, List[int]] = {}
        for i, c in enumerate(labels):
            by_class.setdefault(int(c), []).append(i)
        self.classes = sorted(by_class)[: num_class if num_class is not None else None]
        self.by_class = by_class

    def __iter__(self):
        rng = random.Random(self.seed)
        classes = list(self.classes)
        if self.shuffle:
            rng.shuffle(classes)
        out = []
        for c in classes:
            members = list(self.by_class[c])
            if self.shuffle:
                rng.shuffle(members)
            out.extend(members[: self.num_val])
        return iter(out if self.num is None else out[: self.num])

    def __len__(self):
        n = sum(min(self.num_val, len(self.by_class[c])) for c in self.classes)
        return n if self.num is None else min(n, self.num)


def build_sampler(config=None, default_args: Optional[dict] = None, module_type: str = "dataset_sampler",
                  class_name: Optional[str] = None, **kwargs):
    """A sampler from ``{"type": name, ...}``, or from ``class_name`` and keyword arguments; None without either."""
    if config is None and class_name is None:
        return None
    if config is not None:
        return MindFormerRegister.get_instance_from_cfg(dict(config), MindFormerModuleType.DATASET_SAMPLER,
                                                        default_args=default_args)
    return MindFormerRegister.get_instance(module_type, class_name, **kwargs)


from .._submodules import alias_children as _alias_children  # noqa: E402

_alias_children(__name__, ['build_sampler'])
