"""``Pipeline`` base (reference ``pipeline/base_pipeline.py:53``)."""
from ..pipeline import Pipeline  # noqa: F401
BasePipeline = Pipeline

__all__ = ["Pipeline"]
