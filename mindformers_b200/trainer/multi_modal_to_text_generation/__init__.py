"""``MultiModalToTextGenerationTrainer`` (reference ``trainer/multi_modal_to_text_generation``)."""
from ...trainer.base_trainer import MultiModalToTextGenerationTrainer  # noqa: F401

__all__ = ["MultiModalToTextGenerationTrainer"]
