"""``TextGenerationPipeline`` (reference ``pipeline/text_generation_pipeline.py:31``)."""
from ..pipeline import TextGenerationPipeline  # noqa: F401

__all__ = ["TextGenerationPipeline"]
