"""``KeyWordGenDataset`` (reference ``dataset/keyword_gen_dataset.py``)."""
from ..dataset.causal_language_model_dataset import KeyWordGenDataset  # noqa: F401

__all__ = ["KeyWordGenDataset"]
