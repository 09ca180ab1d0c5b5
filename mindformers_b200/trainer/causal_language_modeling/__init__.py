"""``CausalLanguageModelingTrainer`` (reference ``trainer/causal_language_modeling``)."""
from ...trainer.base_trainer import CausalLanguageModelingTrainer  # noqa: F401

__all__ = ["CausalLanguageModelingTrainer"]
