from .base_trainer import BaseTrainer, CausalLanguageModelingTrainer, GeneralTaskTrainer, build_trainer
from .engine import TrainingEngine
from .trainer import Trainer
from .training_args import TrainingArguments
