"""Qwen3 under its reference import path (``mindformers/models/qwen3``)."""
from ...models.families import Qwen3Config, Qwen3ForCausalLM  # noqa: F401

__all__ = ["Qwen3Config", "Qwen3ForCausalLM"]
