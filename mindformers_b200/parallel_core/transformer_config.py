"""``TransformerConfig`` (reference ``parallel_core/transformer_config.py``)."""
from ..parallel.transformer_config import TransformerConfig  # noqa: F401

__all__ = ["TransformerConfig"]
