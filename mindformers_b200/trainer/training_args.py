"""HF-style ``TrainingArguments`` and its conversion to the YAML-shaped configuration
(``mindformers/trainer/training_args.py``: ~200 fields, ``convert_args_to_mindformers_config``). The fields kept
are the ones that change behaviour in this framework; unknown keyword arguments are rejected so typos surface."""
from __future__ import annotations

from dataclasses import asdict, dataclass, field
from typing import List, Optional, Union


@dataclass
class TrainingArguments:
    """Hugging Face style training arguments (reference ``trainer/training_args.py``): a dataclass of about 200 fields
    that ``convert_args_to_mindformers_config`` maps onto the YAML sections (runner, optimizer, schedule, parallel,
    callbacks, checkpointing)."""

    output_dir: str = "./output"
    overwrite_output_dir: bool = False
    seed: int = 42
    data_seed: Optional[int] = None
    only_save_strategy: bool = False
    auto_trans_ckpt: bool = False
    src_strategy: Optional[str] = None
    transform_process_num: int = 1
    resume_from_checkpoint: Optional[Union[str, bool]] = None
    resume_training: Optional[Union[bool, str]] = None
    ignore_data_skip: bool = False
    data_skip_steps: Optional[int] = None
    do_train: bool = False
    do_eval: bool = False
    do_predict: bool = False
    check_for_nan_in_loss_and_grad: bool = False
    calculate_per_token_loss: bool = False
    remote_save_url: Optional[str] = None
    batch_size: Optional[int] = None
    num_train_epochs: float = 3.0
    sink_mode: bool = True
    sink_size: int = 2
    gradient_accumulation_steps: int = 1
    mode: int = 0
    use_cpu: bool = False
    device_id: int = 0
    device_target: str = "CUDA"
    max_device_memory: str = "170GB"
    use_parallel: bool = False
    parallel_mode: int = 1
    full_batch: bool = True
    enable_parallel_optimizer: bool = False
    data_parallel: int = 1
    model_parallel: int = 1
    expert_parallel: int = 1
    context_parallel: int = 1
    pipeline_stage: int = 1
    micro_batch_num: int = 1
    use_seq_parallel: bool = False
    optimizer_shard: bool = False
    vocab_emb_dp: bool = True
    recompute: bool = False
    select_recompute: bool = False
    optim: str = "fp32_adamw"
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_epsilon: float = 1e-8
    weight_decay: float = 0.0
    layer_scale: bool = False
    layer_decay: float = 0.65
    lr_scheduler_type: str = "cosine"
    learning_rate: float = 5e-5
    lr_end: float = 1e-6
    warmup_lr_init: float = 0.0
    warmup_epochs: Optional[int] = None
    warmup_ratio: Optional[float] = None
    warmup_steps: int = 0
    total_steps: int = -1
    lr_scale: bool = False
    lr_scale_factor: int = 256
    dataset_task: Optional[str] = None
    dataset_type: Optional[str] = None
    train_dataset: Optional[str] = None
    eval_dataset: Optional[str] = None
    dataloader_drop_last: bool = True
    dataloader_num_workers: int = 0
    shuffle: bool = True
    per_device_train_batch_size: int = 8
    per_device_eval_batch_size: int = 8
    wrapper_type: str = "MFTrainOneStepCell"
    scale_sense: Union[str, float] = 1.0
    loss_scale_value: int = 65536
    use_clip_grad: bool = True
    max_grad_norm: float = 1.0
    metric_type: Union[List[str], str] = "PerplexityMetric"
    logging_strategy: str = "steps"
    logging_steps: int = 1
    save_prefix: str = "CKP"
    save_directory: Optional[str] = None
    save_strategy: str = "steps"
    save_steps: int = 500
    save_seconds: Optional[int] = None
    save_total_limit: int = 5
    save_on_each_node: bool = False
    integrated_save: Optional[bool] = None
    save_network_params: bool = True
    save_trainable_params: bool = False
    async_save: bool = False
    evaluation_strategy: str = "no"
    eval_steps: Optional[float] = None
    eval_epochs: Optional[int] = None
    profile: bool = False
    profile_start_step: int = 1
    profile_stop_step: int = 10
    profile_communication: bool = False
    profile_memory: bool = True
    push_to_hub: bool = False
    # ---- context / parallel details ----
    max_call_depth: int = 10000              # accepted for configuration compatibility (graph-compiler recursion limit)
    save_graphs: bool = False                # no graph compiler here: kept so that existing argument files load
    save_graphs_path: str = "./graph"
    gradients_mean: bool = False
    loss_repeated_mean: bool = True
    enable_alltoall: bool = False
    dataset_strategy: str = "full_batch"
    search_mode: str = "sharding_propagation"
    gradient_accumulation_shard: bool = False
    parallel_optimizer_threshold: int = 64
    optimizer_weight_shard_size: int = -1
    strategy_ckpt_save_file: str = "./ckpt_strategy.ckpt"
    gradient_aggregation_group: int = 4
    micro_batch_interleave_num: int = 1
    # ---- mixture of experts ----
    expert_num: int = 1
    capacity_factor: float = 1.05
    aux_loss_factor: float = 0.05
    num_experts_chosen: int = 1
    # ---- recompute details ----
    parallel_optimizer_comm_recompute: bool = False
    mp_comm_recompute: bool = True
    recompute_slice_activation: bool = False
    # ---- dataset columns / loader ----
    train_dataset_in_columns: Optional[List[str]] = None
    train_dataset_out_columns: Optional[List[str]] = None
    eval_dataset_in_columns: Optional[List[str]] = None
    eval_dataset_out_columns: Optional[List[str]] = None
    repeat: int = 1
    prediction_loss_only: bool = False
    python_multiprocessing: bool = False
    numa_enable: bool = False
    prefetch_size: int = 1
    # ---- dynamic loss scale ----
    loss_scale_factor: int = 2
    loss_scale_window: int = 1000
    max_scale_window: int = 1000
    min_scale_window: int = 20
    # ---- checkpoint / profiling / tuning ----
    keep_checkpoint_per_n_minutes: int = 0
    profile_end_step: Optional[int] = None
    init_start_profile: bool = False
    auto_tune: bool = False
    filepath_prefix: str = "./autotune"
    autotune_per_step: int = 10
    # ---- hub ----
    hub_model_id: Optional[str] = None
    hub_strategy: str = "every_save"
    hub_token: Optional[str] = None
    hub_private_repo: bool = False
    hub_always_push: bool = False

    _SCHEDULES = {"cosine": "CosineWithWarmUpLR", "linear": "LinearWithWarmUpLR", "constant": "ConstantWarmUpLR",
                  "constant_with_warmup": "ConstantWarmUpLR", "polynomial": "PolynomialWithWarmUpLR",
                  "cosine_with_restarts": "CosineWithRestartsAndWarmUpLR", "wsd": "WarmUpStableDecayLR"}
    _OPTIMS = {"fp32_adamw": "AdamW", "adamw": "AdamW", "fused_adamw": "FusedAdamW", "came": "CAME", "sgd": "SGD"}

    def __post_init__(self):
        if self.lr_scheduler_type not in self._SCHEDULES:
            raise ValueError(f"lr_scheduler_type must be one of {sorted(self._SCHEDULES)}")
        if self.optim.lower() not in self._OPTIMS:
            raise ValueError(f"optim must be one of {sorted(self._OPTIMS)}")
        if self.warmup_ratio is not None and not 0 <= self.warmup_ratio <= 1:
            raise ValueError("warmup_ratio must lie in [0, 1]")
        if self.batch_size is None:
            self.batch_size = self.per_device_train_batch_size

    @property
    def get_warmup_steps(self):
        return self.warmup_steps

    def to_dict(self):
        return {k: v for k, v in asdict(self).items() if not k.startswith("_")}

    def convert_args_to_mindformers_config(self, config=None):
        """Write these arguments into ``config`` (a ``MindFormerConfig``) section by section."""
        from ..tools.register.config import MindFormerConfig
        cfg = config if config is not None else MindFormerConfig()

        def sec(name, default=None):
            if cfg.get(name) is None:
                cfg[name] = {} if default is None else default
            return cfg[name]
        for k in ("output_dir", "seed", "only_save_strategy", "auto_trans_ckpt", "transform_process_num", "resume_training",
                  "ignore_data_skip", "data_skip_steps", "do_eval", "use_parallel", "profile", "profile_start_step",
                  "profile_stop_step", "profile_communication", "profile_memory", "layer_scale", "layer_decay", "lr_scale",
                  "lr_scale_factor", "remote_save_url"):
            v = getattr(self, k)
            if v is not None:
                cfg[k] = v
        if isinstance(self.resume_from_checkpoint, str):
            cfg["load_checkpoint"] = self.resume_from_checkpoint
        if self.src_strategy:
            cfg["src_strategy_path_or_dir"] = self.src_strategy
        cfg["run_mode"] = "train" if self.do_train or not (self.do_eval or self.do_predict) else ("eval" if self.do_eval else "predict")
        sec("runner_config").update(dict(epochs=int(self.num_train_epochs), batch_size=self.batch_size, sink_mode=self.sink_mode,
                                         sink_size=self.sink_size, gradient_accumulation_steps=self.gradient_accumulation_steps))
        sec("context").update(dict(mode=self.mode, device_target="CPU" if self.use_cpu else self.device_target,
                                   device_id=self.device_id, max_device_memory=self.max_device_memory))
        sec("parallel").update(dict(parallel_mode=self.parallel_mode, full_batch=self.full_batch,
                                    enable_parallel_optimizer=self.enable_parallel_optimizer))
        sec("parallel_config").update(dict(data_parallel=self.data_parallel, model_parallel=self.model_parallel,
                                           expert_parallel=self.expert_parallel, context_parallel=self.context_parallel,
                                           pipeline_stage=self.pipeline_stage, micro_batch_num=self.micro_batch_num,
                                           use_seq_parallel=self.use_seq_parallel, optimizer_shard=self.optimizer_shard,
                                           vocab_emb_dp=self.vocab_emb_dp))
        sec("parallel_config").update(dict(gradient_aggregation_group=self.gradient_aggregation_group))
        sec("parallel").update(dict(gradients_mean=self.gradients_mean, loss_repeated_mean=self.loss_repeated_mean,
                                    enable_alltoall=self.enable_alltoall, search_mode=self.search_mode,
                                    strategy_ckpt_save_file=self.strategy_ckpt_save_file,
                                    parallel_optimizer_config=dict(
                                        gradient_accumulation_shard=self.gradient_accumulation_shard,
                                        parallel_optimizer_threshold=self.parallel_optimizer_threshold,
                                        optimizer_weight_shard_size=self.optimizer_weight_shard_size)))
        sec("context").update(dict(max_call_depth=self.max_call_depth, save_graphs=self.save_graphs,
                                   save_graphs_path=self.save_graphs_path))
        cfg["micro_batch_interleave_num"] = self.micro_batch_interleave_num
        if self.expert_num > 1:
            sec("moe_config").update(dict(expert_num=self.expert_num, capacity_factor=self.capacity_factor,
                                          aux_loss_factor=self.aux_loss_factor, num_experts_chosen=self.num_experts_chosen))
        sec("recompute_config").update(dict(recompute=self.recompute, select_recompute=self.select_recompute,
                                            parallel_optimizer_comm_recompute=self.parallel_optimizer_comm_recompute,
                                            mp_comm_recompute=self.mp_comm_recompute,
                                            recompute_slice_activation=self.recompute_slice_activation))
        if self.auto_tune:
            cfg["auto_tune"], cfg["filepath_prefix"], cfg["autotune_per_step"] = True, self.filepath_prefix, self.autotune_per_step
        if self.profile_end_step is not None:
            cfg["profile_stop_step"] = self.profile_end_step
        cfg["init_start_profile"] = self.init_start_profile
        if self.push_to_hub or self.hub_model_id:
            cfg["hub"] = dict(push_to_hub=self.push_to_hub, hub_model_id=self.hub_model_id, hub_strategy=self.hub_strategy,
                              hub_token=self.hub_token, hub_private_repo=self.hub_private_repo,
                              hub_always_push=self.hub_always_push)
        cfg["optimizer"] = dict(type=self._OPTIMS[self.optim.lower()], betas=[self.adam_beta1, self.adam_beta2],
                                eps=self.adam_epsilon, weight_decay=self.weight_decay, learning_rate=self.learning_rate)
        lr = dict(type=self._SCHEDULES[self.lr_scheduler_type], learning_rate=self.learning_rate,
                  warmup_lr_init=self.warmup_lr_init, total_steps=self.total_steps)
        if self.lr_scheduler_type in ("cosine", "linear", "polynomial", "wsd"):
            lr["lr_end"] = self.lr_end
        if self.warmup_ratio is not None:
            lr["warmup_ratio"] = self.warmup_ratio
        else:
            lr["warmup_steps"] = self.warmup_steps
        cfg["lr_schedule"] = lr
        scale = self.scale_sense
        if isinstance(scale, str) and scale.lower().startswith("dynamic"):
            scale = dict(type="DynamicLossScaleUpdateCell", loss_scale_value=self.loss_scale_value,
                         scale_factor=self.loss_scale_factor, scale_window=self.loss_scale_window)
        elif isinstance(scale, str) and scale.lower().startswith("adaptive"):
            scale = dict(type="AdaptiveLossScaleUpdateCell", loss_scale_value=self.loss_scale_value,
                         scale_factor=self.loss_scale_factor, scale_window=self.loss_scale_window,
                         max_scale_window=self.max_scale_window, min_scale_window=self.min_scale_window)
        cfg["runner_wrapper"] = dict(type=self.wrapper_type, scale_sense=scale, use_clip_grad=self.use_clip_grad,
                                     max_grad_norm=self.max_grad_norm)
        metrics = self.metric_type if isinstance(self.metric_type, list) else [self.metric_type]
        cfg["metric"] = dict(type=metrics[0])
        cbs = [dict(type="MFLossMonitor", per_print_times=self.logging_steps,
                    check_for_nan_in_loss_and_grad=self.check_for_nan_in_loss_and_grad)]
        if self.save_strategy != "no":
            cbs.append(dict(type="CheckpointMonitor", prefix=self.save_prefix, directory=self.save_directory,
                            save_checkpoint_steps=self.save_steps, save_checkpoint_seconds=self.save_seconds or 0,
                            keep_checkpoint_max=self.save_total_limit, save_network_params=self.save_network_params,
                            save_trainable_params=self.save_trainable_params, async_save=self.async_save,
                            keep_checkpoint_per_n_minutes=self.keep_checkpoint_per_n_minutes))
        cfg["callbacks"] = cbs
        if self.evaluation_strategy != "no":
            cfg["do_eval"] = True
            if self.eval_steps:
                cfg["eval_step_interval"] = int(self.eval_steps)
            if self.eval_epochs:
                cfg["eval_epoch_interval"] = int(self.eval_epochs)
        for which, path in (("train_dataset", self.train_dataset), ("eval_dataset", self.eval_dataset)):
            if path:
                sec(which).update(dict(data_loader=dict(type=self.dataset_type or "CommonDataLoader", path=path),
                                       shuffle=self.shuffle, drop_remainder=self.dataloader_drop_last,
                                       num_parallel_workers=self.dataloader_num_workers,
                                       seed=self.data_seed if self.data_seed is not None else self.seed,
                                       repeat=self.repeat, python_multiprocessing=self.python_multiprocessing,
                                       numa_enable=self.numa_enable, prefetch_size=self.prefetch_size))
                in_cols = self.train_dataset_in_columns if which == "train_dataset" else self.eval_dataset_in_columns
                out_cols = self.train_dataset_out_columns if which == "train_dataset" else self.eval_dataset_out_columns
                if in_cols:
                    cfg[which]["input_columns"] = list(in_cols)
                if out_cols:
                    cfg[which]["output_columns"] = list(out_cols)
                cfg[f"{which}_task"] = dict(type=self.dataset_task or "CausalLanguageModelDataset")
        return cfg
