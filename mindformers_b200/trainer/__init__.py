from .base_trainer import BaseTrainer, CausalLanguageModelingTrainer, GeneralTaskTrainer, build_trainer
from .engine import TrainingEngine
from .trainer import Trainer
from .training_args import TrainingArguments
from .config_args import (BaseArgsConfig, CheckpointConfig, CloudConfig, ConfigArguments, ContextConfig, DataLoaderConfig,
                          DatasetConfig, LRConfig, MFContextConfig, OptimizerConfig, ParallelConfig,
                          ParallelContextConfig, RunnerConfig, WrapperConfig)
