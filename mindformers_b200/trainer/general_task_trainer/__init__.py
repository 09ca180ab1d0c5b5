"""``GeneralTaskTrainer`` (reference ``trainer/general_task_trainer``)."""
from ...trainer.base_trainer import GeneralTaskTrainer  # noqa: F401

__all__ = ["GeneralTaskTrainer"]
