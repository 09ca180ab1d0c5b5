"""``ModelParallelConfig`` (reference ``parallel_core/model_parallel_config.py``)."""
from ..parallel.transformer_config import ModelParallelConfig  # noqa: F401

__all__ = ["ModelParallelConfig"]
