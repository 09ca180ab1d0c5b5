"""Adapter classes of the reference's ``pet/tuners`` that are not adapters of their own here.

``PetAdapter`` (reference ``pet/tuners/pet_adapter.py:26``) is the base with the freezing rule; ``PrefixTuningAdapter``
and ``Ptuning2Adapter`` (``prefix_tuning_adapter.py``, ``ptuning2_adapter.py:216``) wrap a model with the prefix
encoder of ``pet/prompt.py``; ``AdaAdapter`` / ``AdaLoraAdapter`` exist in the reference as placeholders without an
implementation (``ada_adapter.py``, ``adalora_adapter.py``: 31 lines each) and raise here as there."""
from __future__ import annotations

import fnmatch
from typing import Iterable, Optional

import torch

from .pet_config import PetConfig, PrefixTuningConfig, Ptuning2Config
from .prompt import PrefixTuningModel

_TRAINABLE = {"lora": ("*lora_a*", "*lora_b*", "*lora_*"), "slora": ("*lora_*",),
              "prefixtuning": ("*prefix*",), "ptuning2": ("*prefix*",)}


class PetAdapter:
    """Base class: ``get_pet_model(model, config)`` returns the adapted model; ``freeze_pretrained_model`` leaves only the
    adapter's parameters (plus ``freeze_exclude`` patterns, minus ``freeze_include`` patterns) trainable."""

    @classmethod
    def get_pet_model(cls, model: torch.nn.Module = None, config: PetConfig = None):
        raise NotImplementedError("get_pet_model is implemented by the adapter classes")

    @staticmethod
    def freeze_pretrained_model(model: torch.nn.Module, pet_type, freeze_include: Optional[Iterable[str]] = None,
                                freeze_exclude: Optional[Iterable[str]] = None):
        kind = str(getattr(pet_type, "value", pet_type)).lower()
        keep = tuple(_TRAINABLE.get(kind, ())) + tuple(freeze_exclude or ())
        force = tuple(freeze_include or ())
        for name, p in model.named_parameters():
            trainable = any(fnmatch.fnmatch(name, pat) for pat in keep) and not any(fnmatch.fnmatch(name, pat) for pat in force)
            p.requires_grad_(trainable)
        return model

    @staticmethod
    def freeze_mcore_pretrained_model(model, freeze_include=None, freeze_exclude=None):
        return PetAdapter.freeze_pretrained_model(model, "lora", freeze_include, freeze_exclude)


class PrefixTuningAdapter(PetAdapter):
    @classmethod
    def get_pet_model(cls, model: torch.nn.Module = None, config=None):
        cfg = config if isinstance(config, PrefixTuningConfig) else PrefixTuningConfig(**dict(config or {}))
        return PrefixTuningModel(cfg, model)


class Ptuning2Adapter(PetAdapter):
    @classmethod
    def get_pet_model(cls, model: torch.nn.Module = None, config=None):
        cfg = config if isinstance(config, Ptuning2Config) else Ptuning2Config(**dict(config or {}))
        return PrefixTuningModel(cfg, model)

    @staticmethod
    def add_prefix(prefix_key_value, key: torch.Tensor, value: torch.Tensor, seq_len_dim: int = 2):
        """Prepend the learned prefix keys / values (``prefix_key_value``: a pair, or a tensor whose first axis holds the
        pair) along the sequence axis; returns ``(key, value)``. None leaves both unchanged."""
        if prefix_key_value is None:
            return key, value
        pk, pv = prefix_key_value[0], prefix_key_value[1]
        return (torch.cat((pk.to(key.dtype), key), dim=seq_len_dim), torch.cat((pv.to(value.dtype), value), dim=seq_len_dim))


class AdaAdapter(PetAdapter):
    @classmethod
    def get_pet_model(cls, model=None, config=None):
        raise NotImplementedError("AdaAdapter has no implementation (neither in the reference)")


class AdaLoraAdapter(PetAdapter):
    @classmethod
    def get_pet_model(cls, model=None, config=None):
        raise NotImplementedError("AdaLoraAdapter has no implementation (neither in the reference)")
