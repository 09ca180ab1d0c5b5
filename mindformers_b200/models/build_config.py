"""``build_model_config`` (reference ``models/build_config.py``)."""
from ..models import build_model_config  # noqa: F401

__all__ = ["build_model_config"]
