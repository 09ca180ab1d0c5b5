"""``LlamaConfig`` (reference ``models/llama/llama_config.py``)."""
from ...models.families import LlamaConfig  # noqa: F401
from ...models.llama_legacy import LlamaLegacyConfig  # noqa: F401

__all__ = ["LlamaConfig", "LlamaLegacyConfig"]
