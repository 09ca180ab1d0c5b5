"""``BaseImageProcessor`` (reference ``models/image_processing_utils.py:452``)."""
from ..models.multi_modal import BaseImageProcessor  # noqa: F401

__all__ = ["BaseImageProcessor"]
