"""``BaseModel`` (reference ``models/base_model.py:39``)."""
from ..models import BaseModel  # noqa: F401

__all__ = ["BaseModel"]
