"""Adapted-model wrappers (reference ``pet/models``: ``lora.py``, ``prefix_tuning.py``, ``ptuning2.py``, ``slora.py``)."""
import torch.nn as nn

from ...pet import LoraModel, PrefixTuningModel  # noqa: F401
from ...pet.pet_config import SLoraConfig
from ...pet.slora import SLoraAdapter


class Ptuning2Model(PrefixTuningModel):
    """P-Tuning v2 wrapper: ``PrefixTuningModel`` driven by a ``Ptuning2Config`` (``pre_seq_len``, ``prefix_projection``)."""


class SLoraModel(nn.Module):
    """Multi-adapter inference wrapper (reference ``pet/models/slora.py:29``): replaces the target linears of
    ``base_model`` by banks of ``lora_num`` adapters and routes every sequence of a batch to the adapter named for it
    (``adapter_names[i]``; None = base model). ``config.adapter_path`` names a ``lora_adapter.json`` (``{adapter name:
    directory}``, each directory holding ``adapter_model.safetensors`` with ``<module>.lora_a`` / ``<module>.lora_b``
    tensors) that is loaded at construction."""

    def __init__(self, config: SLoraConfig, base_model: nn.Module):
        super().__init__()
        self.pet_config = config
        self.network = base_model
        self.slora = SLoraAdapter(base_model, config)
        if getattr(config, "adapter_path", None):
            self.load_adapters(config.adapter_path)

    def load_adapters(self, json_path: str):
        import json
        import os

        from safetensors.torch import load_file
        if os.path.isdir(json_path):
            json_path = os.path.join(json_path, "lora_adapter.json")
        with open(json_path) as f:
            table = json.load(f)
        for name, folder in table.items():
            if not os.path.isabs(folder):
                folder = os.path.join(os.path.dirname(json_path), folder)
            self.slora.load_adapter(name, load_file(os.path.join(folder, "adapter_model.safetensors")))
        return sorted(table)

    def _route(self, input_ids, adapter_names):
        if adapter_names is None:
            return
        ids = input_ids if input_ids.dim() == 2 else input_ids.unsqueeze(0)
        self.slora.set_adapter_ids(list(adapter_names), [ids.shape[1]] * ids.shape[0])

    def forward(self, input_ids, *args, adapter_names=None, **kwargs):
        self._route(input_ids, adapter_names)
        try:
            return self.network(input_ids, *args, **kwargs)
        finally:
            if adapter_names is not None:
                self.slora.clear()


__all__ = ["LoraModel", "PrefixTuningModel", "Ptuning2Model", "SLoraModel"]
