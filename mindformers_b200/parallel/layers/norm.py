"""Normalisation layers: ``RMSNorm`` / ``LayerNorm`` and the ``get_norm`` factory.

Reference: ``training_graph/transformer/norm.py`` (``LayerNorm`` :38, ``FusedLayerNorm`` :115,
``RMSNorm`` :175, ``FusedRMSNorm`` :243, factories :300-339). Statistics are fp32, the result is cast
back to the activation dtype. ``RMSNorm.forward`` optionally takes the residual stream and returns
``(normed, new_residual)`` so the residual add of a pre-LN block is fused into the kernel.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...ops import functional as Fn


class RMSNorm(nn.Module):
    """Root-mean-square norm with an optional fused residual add: ``forward(x, residual=None)`` returns ``norm(x +
    residual) * weight`` (and the new residual stream when one was given). fp32 statistics; the CUDA kernel is
    ``ops/csrc/norm.cu`` (reference ``training_graph/transformer/norm.py:243`` ``FusedRMSNorm``)."""

    def __init__(self, config, hidden_size: int, eps: float = 1e-5):
        super().__init__()
        dev = getattr(config, "device", None) or ("cuda" if torch.cuda.is_available() else "cpu")
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(hidden_size, dtype=config.params_dtype, device=dev))
        self.weight.sequence_parallel = bool(config.sequence_parallel)
        self.weight.no_weight_decay = True

    def forward(self, x, residual=None):
        y, h = Fn.rmsnorm(x, self.weight, self.eps, residual)
        if residual is None:
            return y
        return y, h


class LayerNorm(nn.Module):
    """LayerNorm with the same calling convention as ``RMSNorm`` (reference
    ``training_graph/transformer/norm.py:38,115``)."""

    def __init__(self, config, hidden_size: int, eps: float = 1e-5):
        super().__init__()
        dev = getattr(config, "device", None) or ("cuda" if torch.cuda.is_available() else "cpu")
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(hidden_size, dtype=config.params_dtype, device=dev))
        self.bias = nn.Parameter(torch.zeros(hidden_size, dtype=config.params_dtype, device=dev))
        for p in (self.weight, self.bias):
            p.sequence_parallel = bool(config.sequence_parallel)
            p.no_weight_decay = True

    def forward(self, x, residual=None):
        h = x if residual is None else x + residual
        y = F.layer_norm(h.float(), (h.shape[-1],), self.weight.float(), self.bias.float(), self.eps).to(x.dtype)
        if residual is None:
            return y
        return y, h


FusedRMSNorm = RMSNorm
FusedLayerNorm = LayerNorm


def get_norm(config):
    """Class for ``config.normalization`` (``"RMSNorm"``/``"FusedRMSNorm"``/``"LayerNorm"``/``"FusedLayerNorm"``)."""
    name = config.normalization
    if name in ("RMSNorm", "FusedRMSNorm"):
        return RMSNorm
    if name in ("LayerNorm", "FusedLayerNorm"):
        return LayerNorm
    raise ValueError(f"unknown normalization {name!r}")


def build_norm(config, hidden_size=None, eps=None):
    return get_norm(config)(config, hidden_size or config.hidden_size, eps or config.layernorm_epsilon)
