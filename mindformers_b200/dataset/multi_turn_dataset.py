"""``MultiTurnDataset`` (reference ``dataset/multi_turn_dataset.py``)."""
from ..dataset.causal_language_model_dataset import MultiTurnDataset  # noqa: F401

__all__ = ["MultiTurnDataset"]
