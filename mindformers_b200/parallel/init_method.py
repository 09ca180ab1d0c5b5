"""Weight initialisers of the parallel layers.

Reference: ``parallel_core/utils/init_method.py`` (:27-50): ``init_method_normal(sigma)``,
``scaled_init_method_normal(sigma, num_layers)`` = N(0, sigma / sqrt(2 L)) for the layers that write into the residual
stream (attention output projection and the second MLP matrix), and zeros. Each returns a function that fills a tensor
in place and returns it, which is what the layers' ``init_method`` arguments take.
"""
from __future__ import annotations

import contextlib
import math
from typing import Callable

import torch
import torch.nn as nn


class _NormalInit:
    """Picklable ``tensor -> tensor`` initialiser (configurations that hold one can be copied to worker processes)."""

    def __init__(self, std: float):
        self.std = float(std)

    def __call__(self, tensor: torch.Tensor) -> torch.Tensor:
        return nn.init.normal_(tensor, mean=0.0, std=self.std)

    def __repr__(self):
        return f"normal(std={self.std:g})"


class _ZeroInit:
    def __call__(self, tensor: torch.Tensor) -> torch.Tensor:
        return nn.init.zeros_(tensor)

    def __repr__(self):
        return "zeros"


def init_method_normal(sigma: float = 0.02) -> Callable[[torch.Tensor], torch.Tensor]:
    return _NormalInit(sigma)


def scaled_init_method_normal(sigma: float, num_layers: int) -> Callable[[torch.Tensor], torch.Tensor]:
    """N(0, sigma / sqrt(2 * num_layers)): keeps the variance of the residual stream independent of the depth."""
    return _NormalInit(sigma / math.sqrt(2.0 * max(int(num_layers), 1)))


def init_method_zero() -> Callable[[torch.Tensor], torch.Tensor]:
    return _ZeroInit()


@contextlib.contextmanager
def module_rng(base_seed: int, tag: int, device=None):
    """Random-number scope of one building block of a model (embedding, layer ``i``, output layer): the generators are
    forked and seeded from ``(base_seed, tag)`` alone, so the block's initial weights do not depend on what was built
    before it. A pipeline stage that builds layers 16..31 therefore draws the same values for them as a process that
    builds all 32, the same way a tensor-parallel rank initialises the full matrix and keeps its slice. On exit the
    generators continue where they were."""
    cuda = torch.cuda.is_available() and device is not None and str(device).startswith("cuda")
    devices = [torch.cuda.current_device()] if cuda else []
    with torch.random.fork_rng(devices=devices):
        torch.manual_seed((int(base_seed) * 1000003 + int(tag) * 7919 + 12345) % (2 ** 63 - 1))
        yield
