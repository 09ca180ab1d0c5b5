"""``LlamaTokenizerFast`` (reference ``models/llama/llama_tokenizer_fast.py``)."""
from ...models.tokenizers import LlamaTokenizerFast  # noqa: F401

__all__ = ["LlamaTokenizerFast"]
