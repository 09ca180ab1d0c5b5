"""``build_model`` / ``build_network`` (reference ``models/build_model.py:82``)."""
from ..models import build_model, build_network  # noqa: F401

__all__ = ["build_model", "build_network"]
