"""Key mapping onto ``TransformerConfig`` (reference ``parallel_core/transformer_config_utils.py``)."""
from ..parallel.transformer_config_utils import convert_to_transformer_config  # noqa: F401

__all__ = ["convert_to_transformer_config"]
