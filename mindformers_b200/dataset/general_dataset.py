"""``GeneralDataset`` (reference ``dataset/general_dataset.py``)."""
from ..dataset.causal_language_model_dataset import GeneralDataset  # noqa: F401

__all__ = ["GeneralDataset"]
