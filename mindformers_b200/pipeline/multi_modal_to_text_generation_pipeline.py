"""``MultiModalToTextPipeline`` (reference ``pipeline/multi_modal_to_text_generation_pipeline.py``)."""
from ..pipeline import MultiModalToTextPipeline  # noqa: F401

__all__ = ["MultiModalToTextPipeline"]
