"""The Llama family under its reference import path (``mindformers/models/llama``)."""
from ...models.families import LlamaConfig, LlamaForCausalLM  # noqa: F401
from ...models.llama_legacy import LegacyLlamaForCausalLM, LlamaLegacyConfig  # noqa: F401
from ...models.tokenizers import Llama3Tokenizer, LlamaTokenizer, LlamaTokenizerFast  # noqa: F401
from ...models.processing_utils import LlamaProcessor  # noqa: F401

__all__ = ["LegacyLlamaForCausalLM", "Llama3Tokenizer", "LlamaConfig", "LlamaForCausalLM", "LlamaLegacyConfig", "LlamaProcessor", "LlamaTokenizer", "LlamaTokenizerFast"]
