"""Activation zoo (``mindformers/modules/activation.py``, ``parallel_core/training_graph/activation.py:27-205``)."""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as Fn


class GELU(nn.Module):
    """GELU, exact (erf) or tanh approximation."""

    def __init__(self, approximate: bool = True):
        super().__init__()
        self.approximate = "tanh" if approximate else "none"

    def forward(self, x):
        return F.gelu(x, approximate=self.approximate)


class FastGelu(nn.Module):
    """``x * sigmoid(1.702 x)``."""

    def forward(self, x):
        return x * torch.sigmoid(1.702 * x)


class SiLU(nn.Module):
    """``x * sigmoid(x)``."""

    def forward(self, x):
        return F.silu(x)


class SwiGLU(nn.Module):
    """``silu(x[..., :F]) * x[..., F:]`` (the fused sm_100a kernel on CUDA bf16)."""

    def forward(self, x):
        return Fn.swiglu(x)


class LeakyReLU(nn.LeakyReLU):
    """Leaky ReLU with slope ``alpha`` for negative inputs."""

    pass


class LogSoftmax(nn.LogSoftmax):
    """Log-softmax over ``axis``."""

    pass


_TABLE = {"gelu": GELU, "fast_gelu": FastGelu, "fastgelu": FastGelu, "silu": SiLU, "swish": SiLU, "swiglu": SwiGLU,
          "relu": nn.ReLU, "relu6": nn.ReLU6, "tanh": nn.Tanh, "sigmoid": nn.Sigmoid, "leakyrelu": LeakyReLU,
          "elu": nn.ELU, "softplus": nn.Softplus, "hswish": nn.Hardswish, "hsigmoid": nn.Hardsigmoid, "logsoftmax": LogSoftmax}


def get_activation(name, *args, **kwargs):
    if name is None:
        return None
    key = str(name).lower()
    if key not in _TABLE:
        raise KeyError(f"activation {name!r} is not available; choose from {sorted(_TABLE)}")
    cls = _TABLE[key]
    return cls(*args, **kwargs) if key == "logsoftmax" and (args or kwargs) else (cls(dim=-1) if key == "logsoftmax" else cls(*args, **kwargs))
