"""``LlamaForCausalLM`` (reference ``models/llama/llama.py:408``)."""
from ...models.families import LlamaForCausalLM  # noqa: F401
from ...models.llama_legacy import LegacyLlamaForCausalLM  # noqa: F401

__all__ = ["LegacyLlamaForCausalLM", "LlamaForCausalLM"]
