from .base_trainer import BaseTrainer, CausalLanguageModelingTrainer, GeneralTaskTrainer, build_trainer
from .engine import TrainingEngine
from .trainer import Trainer
from .training_args import TrainingArguments
from .config_args import (BaseArgsConfig, CheckpointConfig, CloudConfig, ConfigArguments, ContextConfig, DataLoaderConfig,
                          DatasetConfig, LRConfig, MFContextConfig, OptimizerConfig, ParallelConfig,
                          ParallelContextConfig, RunnerConfig, WrapperConfig)

from .._submodules import keep_functions as _keep_functions  # noqa: E402

_keep_functions(__name__, ('build_trainer',))
