"""``build_trainer`` (reference ``trainer/build_trainer.py``)."""
from ..trainer import build_trainer  # noqa: F401

__all__ = ["build_trainer"]
