"""``pipeline()`` factory (reference ``pipeline/pipeline.py:59``)."""
from ..pipeline import pipeline, SUPPORTED_TASKS  # noqa: F401

__all__ = ["SUPPORTED_TASKS", "pipeline"]
