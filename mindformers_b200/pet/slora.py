"""S-LoRA: many adapters resident at once, chosen per request at inference time
(``mindformers/pet/tuners/slora_adapter.py:37-574``). Adapter weights are stacked ``[n_adapters + 1, ...]`` with slot 0
all-zero (= no adapter); ``set_adapter_ids`` gives one adapter slot per token of the flattened batch and the layer
gathers each token's ``A`` / ``B`` by that index (two batched matmuls of rank-``r`` width)."""
from __future__ import annotations

import re
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn as nn

from ..parallel.layers.tensor_parallel import ColumnParallelLinear, LinearNoTP, RowParallelLinear
from .pet_config import SLoraConfig


class SLoraLinear(nn.Module):
    """A linear layer with a bank of LoRA pairs: every row of the batch adds the low-rank update of the adapter its
    request selected (index 0 = no adapter)."""

    def __init__(self, base: nn.Module, num_adapters: int, rank: int, alpha: float):
        super().__init__()
        self.base = base
        out_f, in_f = base.weight.shape
        dev, dt = base.weight.device, base.weight.dtype
        self.scaling = alpha / rank
        self.register_buffer("lora_a", torch.zeros(num_adapters + 1, rank, in_f, dtype=dt, device=dev))
        self.register_buffer("lora_b", torch.zeros(num_adapters + 1, out_f, rank, dtype=dt, device=dev))
        self.token_adapter: Optional[torch.Tensor] = None

    @property
    def weight(self):
        return self.base.weight

    def forward(self, x, *args, **kwargs):
        y, bias = self.base(x, *args, **kwargs)
        idx = self.token_adapter
        if idx is None or not bool((idx > 0).any()):
            return y, bias
        a = self.lora_a.index_select(0, idx)                  # [T, r, in]
        b = self.lora_b.index_select(0, idx)                  # [T, out, r]
        h = torch.bmm(a, x.unsqueeze(-1))                     # [T, r, 1]
        d = torch.bmm(b, h).squeeze(-1) * self.scaling
        return y + d.to(y.dtype), bias


class SLoraAdapter:
    """Loads a directory of LoRA adapters into ``SLoraLinear`` banks and routes requests to them by ``adapter_ids``
    (reference ``pet/tuners/slora_adapter.py:37-574``)."""

    def __init__(self, model: nn.Module, config: SLoraConfig):
        self.model, self.config = model, config
        self.names: Dict[str, int] = {}
        self.layers: List[SLoraLinear] = []
        pattern = re.compile(config.target_modules)
        self._replace(model, pattern, "")
        if not self.layers:
            raise ValueError(f"target_modules {config.target_modules!r} matched no linear layer")

    def _replace(self, module, pattern, prefix):
        for name, child in list(module.named_children()):
            full = f"{prefix}.{name}" if prefix else name
            if isinstance(child, (ColumnParallelLinear, RowParallelLinear, LinearNoTP)) and child.weight is not None \
                    and pattern.fullmatch(full):
                if getattr(child, "tp", 1) > 1:
                    raise NotImplementedError("multi-adapter inference is implemented for tensor-parallel size 1")
                wrapped = SLoraLinear(child, self.config.lora_num, self.config.lora_rank, self.config.lora_alpha)
                wrapped.qualified_name = full
                setattr(module, name, wrapped)
                self.layers.append(wrapped)
            else:
                self._replace(child, pattern, full)

    def load_adapter(self, adapter_name: str, state: Dict[str, torch.Tensor]) -> int:
        """Install ``{<module name>.lora_a, <module name>.lora_b}`` tensors under ``adapter_name``; returns its slot."""
        slot = self.names.get(adapter_name)
        if slot is None:
            slot = len(self.names) + 1
            if slot > self.config.lora_num:
                raise ValueError(f"only {self.config.lora_num} adapter slots were allocated")
            self.names[adapter_name] = slot
        for layer in self.layers:
            a = state.get(f"{layer.qualified_name}.lora_a")
            b = state.get(f"{layer.qualified_name}.lora_b")
            if a is not None and b is not None:
                layer.lora_a[slot].copy_(a.to(layer.lora_a.dtype))
                layer.lora_b[slot].copy_(b.to(layer.lora_b.dtype))
        return slot

    def set_adapter_ids(self, adapter_names: Sequence[Optional[str]], tokens_per_sequence: Sequence[int]):
        """``adapter_names[i]`` (``None`` = base model) applies to the ``tokens_per_sequence[i]`` tokens of sequence
        ``i``."""
        dev = self.layers[0].lora_a.device
        slots = torch.tensor([self.names.get(n, 0) if n else 0 for n in adapter_names], device=dev)
        idx = torch.repeat_interleave(slots, torch.tensor(list(tokens_per_sequence), device=dev))
        for layer in self.layers:
            layer.token_adapter = idx

    def clear(self):
        for layer in self.layers:
            layer.token_adapter = None
