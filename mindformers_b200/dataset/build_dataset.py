"""``build_dataset`` (reference ``dataset/build_dataset.py``)."""
from ..dataset.causal_language_model_dataset import build_dataset, build_dataset_loader  # noqa: F401

__all__ = ["build_dataset", "build_dataset_loader"]
