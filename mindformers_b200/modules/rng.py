"""RNG tracker with tensor-parallel forked seeds (``parallel_core/inference/tensor_parallel/random.py:47-140``):
dropout inside tensor-parallel regions must differ across TP ranks, everything else must agree."""
from __future__ import annotations

import contextlib
from typing import Dict

import torch

from ..parallel import parallel_state as ps

_MODEL_PARALLEL = "model-parallel-rng"
_DATA_PARALLEL = "data-parallel-rng"


class CudaRNGStatesTracker:
    """Named random-number states (reference ``inference/tensor_parallel/random.py:47``): ``fork(name)`` runs a block
    under the state registered for ``name`` so that tensor-parallel ranks draw different dropout masks and identical
    initial weights."""

    def __init__(self):
        self.states: Dict[str, torch.Tensor] = {}
        self.seeds = set()

    def reset(self):
        self.states.clear()
        self.seeds.clear()

    def _get(self):
        return torch.cuda.get_rng_state() if torch.cuda.is_available() else torch.get_rng_state()

    def _set(self, s):
        (torch.cuda.set_rng_state if torch.cuda.is_available() else torch.set_rng_state)(s)

    def add(self, name: str, seed: int):
        if seed in self.seeds:
            raise ValueError(f"seed {seed} already exists")
        if name in self.states:
            raise ValueError(f"rng state {name} already exists")
        self.seeds.add(seed)
        keep = self._get()
        (torch.cuda.manual_seed if torch.cuda.is_available() else torch.manual_seed)(seed)
        self.states[name] = self._get()
        self._set(keep)

    @contextlib.contextmanager
    def fork(self, name: str = _MODEL_PARALLEL):
        if name not in self.states:
            raise KeyError(f"rng state {name} was not added")
        keep = self._get()
        self._set(self.states[name])
        try:
            yield
        finally:
            self.states[name] = self._get()
            self._set(keep)


_TRACKER = CudaRNGStatesTracker()


def get_rng_tracker() -> CudaRNGStatesTracker:
    return _TRACKER


def model_parallel_manual_seed(seed: int):
    """Default generator: ``seed`` (same on all TP ranks); tracked model-parallel generator: ``seed + 2718 + tp_rank``.
    Default generator: ``seed`` (same on all TP ranks); tracked model-parallel generator: ``seed + 2718 + tp_rank``."""
    _TRACKER.reset()
    torch.manual_seed(seed)
    _TRACKER.add(_DATA_PARALLEL, seed + 1)
    _TRACKER.add(_MODEL_PARALLEL, seed + 2718 + ps.get_tensor_model_parallel_rank())
