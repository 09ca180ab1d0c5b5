"""Processor bases (reference ``models/base_processor.py``)."""
from ..models.processing_utils import BaseProcessor  # noqa: F401
from ..models.multi_modal import BaseImageProcessor  # noqa: F401

__all__ = ["BaseImageProcessor", "BaseProcessor"]
