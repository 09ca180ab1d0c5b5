"""Qwen2 under its reference import path (``mindformers/models/qwen2``)."""
from ...models.families import Qwen2Config, Qwen2ForCausalLM  # noqa: F401
from ...models.tokenizers import Qwen2Tokenizer  # noqa: F401

__all__ = ["Qwen2Config", "Qwen2ForCausalLM", "Qwen2Tokenizer"]
