"""``Trainer``: the user-facing object behind ``run_mindformer.py`` and the Python API.

``Trainer(args=<yaml path | MindFormerConfig | TrainingArguments>, task=..., model=..., train_dataset=...,
callbacks=...)`` then ``train() / finetune() / evaluate() / predict()`` — the surface of
``mindformers/trainer/trainer.py:180-197,360,489,628,712``. Construction order follows the reference:
configuration → parallel settings → seed → output directories → task trainer → callbacks.
"""
from __future__ import annotations

import copy
import os
from typing import Callable, List, Optional, Union

import torch

from ..checkpoint.resume import get_resume_checkpoint
from ..core.callback import Callback
from ..core.context import build_context, is_context_built
from ..tools.logger import get_logger
from ..tools.register.config import MindFormerConfig
from ..tools.register.template import ConfigTemplate
from ..tools.utils import get_output_root_path, set_output_path
from .base_trainer import build_trainer
from .config_args import ConfigArguments
from .training_args import TrainingArguments

logger = get_logger()

DEFAULT_TASK_CONFIG = {
    "trainer": {"type": "CausalLanguageModelingTrainer"},
    "runner_config": {"epochs": 1, "batch_size": 1},
    "optimizer": {"type": "AdamW", "betas": [0.9, 0.95], "learning_rate": 1e-4, "weight_decay": 0.0},
    "lr_schedule": {"type": "CosineWithWarmUpLR", "learning_rate": 1e-4, "warmup_ratio": 0.0, "total_steps": -1},
    "callbacks": [{"type": "MFLossMonitor"}],
}


class Trainer:
    """High-level entry point (reference ``trainer/trainer.py:180-325``): ``Trainer(args=config file | dict |
    TrainingArguments, task=..., model=..., train_dataset=..., eval_dataset=..., callbacks=...)`` then ``train()``,
    ``finetune()``, ``evaluate()``, ``predict()``. Builds the context, the parallel groups, the task trainer
    registered for ``task`` and hands it the merged configuration."""

    def __init__(self, args: Optional[Union[str, dict, MindFormerConfig, TrainingArguments]] = None, task: str = "general",
                 model=None, model_name: Optional[str] = None, tokenizer=None, train_dataset=None, eval_dataset=None,
                 data_collator: Optional[Callable] = None, optimizers=None, compute_metrics=None,
                 callbacks: Optional[Union[Callback, List[Callback]]] = None, eval_callbacks=None,
                 pet_method: str = "", image_processor=None, audio_processor=None, save_config: bool = False,
                 reset_model: bool = False):
        self.task, self.model, self.model_name, self.tokenizer = task, model, model_name, tokenizer
        self.train_dataset, self.eval_dataset = train_dataset, eval_dataset
        self.compute_metrics = compute_metrics
        self.callbacks = [callbacks] if isinstance(callbacks, Callback) else callbacks
        self.config = self._init_config(args)
        if not is_context_built():
            build_context(self.config)
        if self.config.get("output_dir"):
            set_output_path(self.config["output_dir"])
        self.trainer = build_trainer(self.config.get("trainer"))
        if pet_method or (self.config.get("model") or {}).get("model_config", {}).get("pet_config"):
            self._pet = pet_method or self.config["model"]["model_config"]["pet_config"].get("pet_type")
        if save_config:
            self.config.dump(os.path.join(get_output_root_path(), "run_config.yaml"))
        self.state = None

    # ---------------------------------------------------------------------------------------------
    def _init_config(self, args) -> MindFormerConfig:
        if isinstance(args, TrainingArguments):
            cfg = MindFormerConfig(copy.deepcopy(DEFAULT_TASK_CONFIG))
            args.convert_args_to_mindformers_config(cfg)
        elif isinstance(args, ConfigArguments):
            cfg = MindFormerConfig(copy.deepcopy(DEFAULT_TASK_CONFIG))
            cfg.merge_from_dict(args.to_config())
        elif isinstance(args, str):
            cfg = MindFormerConfig(args)
        elif isinstance(args, dict):
            cfg = args if isinstance(args, MindFormerConfig) else MindFormerConfig(copy.deepcopy(dict(args)))
        elif args is None:
            cfg = MindFormerConfig(copy.deepcopy(DEFAULT_TASK_CONFIG))
        else:
            raise TypeError(f"args must be a path, a mapping or TrainingArguments, got {type(args).__name__}")
        cfg.setdefault("run_mode", "train")
        ConfigTemplate.apply_template(cfg)
        return cfg

    def set_parallel_config(self, data_parallel=1, model_parallel=1, context_parallel=1, expert_parallel=1, pipeline_stage=1,
                            micro_batch_interleave_num=1, micro_batch_num=1, use_seq_parallel=False, optimizer_shard=False,
                            gradient_aggregation_group=4, vocab_emb_dp=True):
        self.config["parallel_config"].update(dict(
            data_parallel=data_parallel, model_parallel=model_parallel, context_parallel=context_parallel,
            expert_parallel=expert_parallel, pipeline_stage=pipeline_stage, micro_batch_num=micro_batch_num,
            use_seq_parallel=use_seq_parallel, optimizer_shard=optimizer_shard,
            gradient_aggregation_group=gradient_aggregation_group, vocab_emb_dp=vocab_emb_dp))
        self.config["micro_batch_interleave_num"] = micro_batch_interleave_num

    def set_recompute_config(self, recompute=False, parallel_optimizer_comm_recompute=False, select_recompute=False,
                             mp_comm_recompute=True, recompute_slice_activation=False):
        self.config["recompute_config"].update(dict(
            recompute=recompute, parallel_optimizer_comm_recompute=parallel_optimizer_comm_recompute,
            select_recompute=select_recompute, mp_comm_recompute=mp_comm_recompute,
            recompute_slice_activation=recompute_slice_activation))

    # ---------------------------------------------------------------------------------------------
    def _resolve_resume(self, train_checkpoint, resume_training):
        cfg = self.config
        if train_checkpoint not in (None, False):
            cfg["load_checkpoint"] = train_checkpoint if isinstance(train_checkpoint, str) else cfg.get("load_checkpoint")
        if resume_training is not None:
            cfg["resume_training"] = resume_training
        path = cfg.get("load_checkpoint")
        if cfg.get("resume_training") and path and os.path.isdir(path):
            point = get_resume_checkpoint(path, cfg["resume_training"])
            if point is None:
                logger.warning("resume_training is set but %s holds no complete checkpoint; starting fresh", path)
                cfg["load_checkpoint"], cfg["resume_training"] = "", False

    def train(self, train_checkpoint=False, resume_from_checkpoint=None, resume_training=None, ignore_data_skip=None,
              data_skip_steps=None, auto_trans_ckpt=None, src_strategy=None, transform_process_num=None, do_eval: bool = False):
        cfg = self.config
        cfg["run_mode"] = cfg.get("run_mode") or "train"
        if resume_from_checkpoint is not None:
            train_checkpoint = resume_from_checkpoint
        self._resolve_resume(train_checkpoint, resume_training)
        if ignore_data_skip is not None:
            cfg["ignore_data_skip"] = ignore_data_skip
        if data_skip_steps is not None:
            cfg["data_skip_steps"] = data_skip_steps
        cbs = self.callbacks
        if do_eval or cfg.get("do_eval"):
            from ..core.callback import EvalCallBack
            extra = EvalCallBack(lambda: self.evaluate(), step_interval=cfg.get("eval_step_interval", 100),
                                 epoch_interval=cfg.get("eval_epoch_interval", -1))
            built = self.trainer.create_callbacks(cfg, {"global_batch_size": self.trainer.global_batch_size(cfg)})
            cbs = (cbs or built) + [extra]
        self.state = self.trainer.training_process(cfg, network=self.model, dataset=self.train_dataset, callbacks=cbs)
        return self.state

    def finetune(self, finetune_checkpoint=False, resume_from_checkpoint=None, resume_training=None, **kw):
        self.config["run_mode"] = "finetune"
        return self.train(train_checkpoint=finetune_checkpoint, resume_from_checkpoint=resume_from_checkpoint,
                          resume_training=resume_training, **kw)

    def evaluate(self, eval_dataset=None, eval_checkpoint=False, **kw):
        if isinstance(eval_checkpoint, str):
            self.config["load_checkpoint"] = eval_checkpoint
        model = self.model if self.model is not None else (self.trainer.engine.model if self.trainer.engine else None)
        return self.trainer.evaluate_process(self.config, network=model, dataset=eval_dataset or self.eval_dataset,
                                             metric=self.compute_metrics, **kw)

    def predict(self, predict_checkpoint=None, input_data=None, batch_size=None, **kw):
        if isinstance(predict_checkpoint, str):
            self.config["load_checkpoint"] = predict_checkpoint
        if batch_size:
            self.config["predict_batch_size"] = batch_size
        return self.trainer.predict_process(self.config, input_data=input_data, network=self.model, tokenizer=self.tokenizer, **kw)

    def save_model(self, output_dir: Optional[str] = None):
        model = self.model if self.model is not None else self.trainer.engine.model
        out = output_dir or os.path.join(get_output_root_path(), "saved_model")
        if hasattr(model, "save_pretrained"):
            model.save_pretrained(out)
        else:
            from ..checkpoint.io import save_pretrained_dir
            save_pretrained_dir(model, out)
        if self.tokenizer is not None and hasattr(self.tokenizer, "save_pretrained"):
            self.tokenizer.save_pretrained(out)
        return out

    def push_to_hub(self, *a, **kw):
        raise RuntimeError("no network access from this environment: use save_model() and upload the directory yourself")
