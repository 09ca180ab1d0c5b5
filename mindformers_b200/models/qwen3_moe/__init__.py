"""Qwen3-MoE under its reference import path (``mindformers/models/qwen3_moe``)."""
from ...models.families import Qwen3MoeConfig, Qwen3MoeForCausalLM  # noqa: F401

__all__ = ["Qwen3MoeConfig", "Qwen3MoeForCausalLM"]
