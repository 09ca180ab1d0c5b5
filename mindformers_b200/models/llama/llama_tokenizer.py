"""``LlamaTokenizer`` (reference ``models/llama/llama_tokenizer.py``)."""
from ...models.tokenizers import LlamaTokenizer  # noqa: F401

__all__ = ["LlamaTokenizer"]
