"""``build_processor`` (reference ``models/build_processor.py``)."""
from ..models.processing_utils import build_processor  # noqa: F401

__all__ = ["build_processor"]
