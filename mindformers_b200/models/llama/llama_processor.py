"""``LlamaProcessor`` (reference ``models/llama/llama_processor.py``)."""
from ...models.processing_utils import LlamaProcessor  # noqa: F401

__all__ = ["LlamaProcessor"]
