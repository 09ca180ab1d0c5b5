"""LoRA for the tensor-parallel linear layers.

Reference: ``training_graph/tensor_parallel/lora_layers.py`` (``ColumnParallelLinearWithLoRA`` :56,
``RowParallelLinearWithLoRA`` :234: ``lora_a``/``lora_b``, ``scaling = alpha / rank``, dropout on the LoRA input) and
``pet/tuners/lora_adapter.py:59,153`` (recursive replacement by regular expression, base weights frozen).

Sharding keeps the adapter's communication at rank-``r`` width:
* column-parallel base (``W [out/tp, in]``): ``lora_a [r, in]`` replicated, ``lora_b [out/tp, r]`` sharded like the base;
  under sequence parallelism the ``[T/tp, r]`` product is all-gathered, never the hidden states a second time;
* row-parallel base (``W [out, in/tp]``): ``lora_a [r, in/tp]`` sharded, ``lora_b [out, r]`` replicated; the ``[T, r]``
  partial products are all-reduced (reduce-scattered under sequence parallelism).
"""
from __future__ import annotations

import math
import re
from typing import Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..parallel import mappings as M
from ..parallel.layers.tensor_parallel import ColumnParallelLinear, LinearNoTP, RowParallelLinear
from .pet_config import LoraConfig


def _dtype(name):
    return name if isinstance(name, torch.dtype) else getattr(torch, str(name).replace("torch.", ""))


class LoRALinear(nn.Module):
    """Wraps a (column / row / plain) linear layer; returns ``(output, bias)`` like the wrapped layer."""

    def __init__(self, base: nn.Module, rank: int = 8, alpha: float = 16, dropout: float = 0.0,
                 param_dtype=torch.float32, a_init: str = "normal"):
        super().__init__()
        self.base = base
        self.rank, self.scaling = rank, alpha / rank
        self.dropout = nn.Dropout(dropout) if dropout > 0 else None
        w = base.weight
        out_f, in_f = w.shape
        dev = w.device
        self.kind = "column" if isinstance(base, ColumnParallelLinear) else "row" if isinstance(base, RowParallelLinear) else "plain"
        self.tp = getattr(base, "tp", 1)
        self.sp = bool(getattr(base, "sequence_parallel", False)) and self.tp > 1
        a = torch.empty(rank, in_f, dtype=param_dtype, device=dev)
        if a_init == "kaiming":
            nn.init.kaiming_uniform_(a, a=math.sqrt(5))
        else:
            a.normal_(0.0, 0.01)
        self.lora_a = nn.Parameter(a)
        self.lora_b = nn.Parameter(torch.zeros(out_f, rank, dtype=param_dtype, device=dev))
        if self.tp > 1:
            if self.kind == "column":
                self.lora_b.tensor_model_parallel, self.lora_b.partition_dim = True, 0
                self.lora_a.sequence_parallel = self.sp
            elif self.kind == "row":
                self.lora_a.tensor_model_parallel, self.lora_a.partition_dim = True, 1
                self.lora_b.sequence_parallel = self.sp
        for p in base.parameters():
            p.requires_grad_(False)
        self.merged = False

    @property
    def weight(self):
        return self.base.weight

    def _delta(self, x):
        xd = x if self.dropout is None else self.dropout(x)
        a, b = self.lora_a.to(x.dtype), self.lora_b.to(x.dtype)
        if self.kind == "row" and not self.base.input_is_parallel and self.tp > 1:
            xd = xd.chunk(self.tp, dim=-1)[self.base.rank]
        h = F.linear(xd, a)                                   # [T(/tp), r]
        if self.tp > 1:
            if self.kind == "column":
                h = M.gather_from_sequence_parallel_region(h) if self.sp else M.copy_to_tensor_model_parallel_region(h)
            elif self.kind == "row":
                h = M.reduce_scatter_to_sequence_parallel_region(h) if self.sp else M.reduce_from_tensor_model_parallel_region(h)
        return F.linear(h, b) * self.scaling

    def forward(self, x, *args, **kwargs):
        y, bias = self.base(x, *args, **kwargs)
        if not self.merged:
            d = self._delta(x)
            if self.kind == "column" and self.tp > 1 and self.base.gather_output:
                d = M.gather_from_tensor_model_parallel_region(d)
            y = y + d
        return y, bias

    @torch.no_grad()
    def merge(self):
        """Fold ``scaling · B A`` into the base weight (inference without the extra matmuls)."""
        if not self.merged:
            self.base.weight.add_((self.lora_b.float() @ self.lora_a.float() * self.scaling).to(self.base.weight.dtype))
            self.merged = True

    @torch.no_grad()
    def unmerge(self):
        if self.merged:
            self.base.weight.sub_((self.lora_b.float() @ self.lora_a.float() * self.scaling).to(self.base.weight.dtype))
            self.merged = False


class ColumnParallelLinearWithLoRA(LoRALinear):
    """Column-parallel linear layer with a LoRA branch: ``lora_a`` replicated, ``lora_b`` split like the weight
    (reference ``training_graph/tensor_parallel/lora_layers.py:56``). Builds the base layer itself."""

    def __init__(self, input_size: int, output_size: int, *, config, lora_rank: int = 8, lora_alpha: float = 16,
                 lora_dropout: float = 0.0, lora_a_init: str = "normal", **base_kwargs):
        super().__init__(ColumnParallelLinear(input_size, output_size, config=config, **base_kwargs), lora_rank,
                         lora_alpha, lora_dropout, a_init=lora_a_init)


class RowParallelLinearWithLoRA(LoRALinear):
    """Row-parallel linear layer with a LoRA branch: ``lora_a`` split like the weight, ``lora_b`` replicated
    (reference ``training_graph/tensor_parallel/lora_layers.py:234``)."""

    def __init__(self, input_size: int, output_size: int, *, config, lora_rank: int = 8, lora_alpha: float = 16,
                 lora_dropout: float = 0.0, lora_a_init: str = "normal", **base_kwargs):
        super().__init__(RowParallelLinear(input_size, output_size, config=config, **base_kwargs), lora_rank,
                         lora_alpha, lora_dropout, a_init=lora_a_init)


class LoraAdapter:
    """``get_pet_model(model, config)``: replaces the linear layers matched by ``target_modules`` with their LoRA
    versions and freezes everything else (reference ``pet/tuners/lora_adapter.py:59,153``
    ``recursive_replace_dense_cell``)."""

    @staticmethod
    def recursive_replace_dense_cell(module: nn.Module, config: LoraConfig, prefix: str = "") -> int:
        """Replace every linear layer whose qualified name matches ``config.target_modules``; returns the count."""
        pattern = re.compile(config.target_modules)
        exclude = [re.compile(p) for p in (config.exclude_layers or [])]
        count = 0
        for name, child in list(module.named_children()):
            full = f"{prefix}.{name}" if prefix else name
            if isinstance(child, (ColumnParallelLinear, RowParallelLinear, LinearNoTP)) and child.weight is not None \
                    and pattern.fullmatch(full) and not any(e.search(full) for e in exclude):
                setattr(module, name, LoRALinear(child, config.lora_rank, config.lora_alpha, config.lora_dropout,
                                                 _dtype(config.param_init_type), "normal" if config.lora_a_init == "normal" else "kaiming"))
                count += 1
            elif not isinstance(child, LoRALinear):
                count += LoraAdapter.recursive_replace_dense_cell(child, config, full)
        return count

    @classmethod
    def get_pet_model(cls, model: nn.Module, config: LoraConfig) -> nn.Module:
        for p in model.parameters():
            p.requires_grad_(False)
        n = cls.recursive_replace_dense_cell(model, config)
        if n == 0:
            raise ValueError(f"target_modules {config.target_modules!r} matched no linear layer")
        keep = [re.compile(p) for p in (config.freeze_exclude or [])]
        for name, p in model.named_parameters():
            if "lora_a" in name or "lora_b" in name or any(k.search(name) for k in keep):
                p.requires_grad_(True)
        return model


class LoraModel(nn.Module):
    """``LoraModel(config, base_model)``: the base model with LoRA layers inserted and everything else frozen."""

    def __init__(self, config: LoraConfig, base_model: nn.Module):
        super().__init__()
        self.config = base_model.config if hasattr(base_model, "config") else None
        self.pet_config = config if isinstance(config, LoraConfig) else LoraConfig(**dict(config))
        self.network = LoraAdapter.get_pet_model(base_model, self.pet_config)

    def forward(self, *a, **kw):
        return self.network(*a, **kw)

    def generate(self, *a, **kw):
        return self.network.generate(*a, **kw)

    def merge_and_unload(self):
        merge_lora_weights(self.network)
        return self.network


def merge_lora_weights(model: nn.Module):
    for m in model.modules():
        if isinstance(m, LoRALinear):
            m.merge()


def lora_state_dict(model: nn.Module) -> Dict[str, torch.Tensor]:
    """Only the adapter tensors (what ``checkpoint_trainable`` holds for a LoRA run)."""
    return {n: p.detach() for n, p in model.named_parameters() if "lora_a" in n or "lora_b" in n}
