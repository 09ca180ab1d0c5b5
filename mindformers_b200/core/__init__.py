"""Optimizers, learning-rate schedules, losses, metrics, callbacks and the run context."""
from .callback import (CheckpointMonitor, EvalCallBack, MFLossMonitor, ProfileMonitor, SummaryMonitor,
                       TrainingStateMonitor, build_callback)
from .clip_grad import ClipGradNorm
from .context import build_context, get_context, init_context, set_context
from .loss import CrossEntropyLoss, build_loss
from .lr import (ConstantWarmUpLR, CosineAnnealingLR, CosineAnnealingWarmRestarts, CosineWithRestartsAndWarmUpLR,
                 CosineWithWarmUpLR, LearningRateWiseLayer, LinearWithWarmUpLR, PolynomialWithWarmUpLR,
                 WarmUpStableDecayLR, build_lr)
from .metric import ADGENMetric, EmF1Metric, EntityScore, PerplexityMetric, PromptAccMetric, build_metric
from .optim import CAME, AdamW, FusedAdamW, build_optim
from .parallel_config import build_parallel_config
