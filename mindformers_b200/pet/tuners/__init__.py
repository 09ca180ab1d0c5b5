"""Adapters (reference ``pet/tuners``: ``lora_adapter.py:59``, ``slora_adapter.py``, prefix / p-tuning)."""
from ...pet import LoraAdapter, SLoraAdapter, PrefixEncoder  # noqa: F401

__all__ = ["LoraAdapter", "PrefixEncoder", "SLoraAdapter"]
