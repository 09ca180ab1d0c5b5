"""Adapters (reference ``pet/tuners``: ``lora_adapter.py:59``, ``slora_adapter.py``, prefix / p-tuning)."""
from ...pet import LoraAdapter, SLoraAdapter, PrefixEncoder  # noqa: F401
from ...pet.adapters import AdaAdapter, AdaLoraAdapter, PetAdapter, PrefixTuningAdapter, Ptuning2Adapter  # noqa: F401
from ...pet.slora import SLoraLinear  # noqa: F401

Ptuning2Encoder = PrefixEncoder

__all__ = ["AdaAdapter", "AdaLoraAdapter", "LoraAdapter", "PetAdapter", "PrefixEncoder", "PrefixTuningAdapter", "Ptuning2Adapter",
           "Ptuning2Encoder", "SLoraAdapter", "SLoraLinear"]
