"""Typed mirrors of the YAML sections, for building a trainer configuration in code.

Each class lists the keys of one YAML section (``ContextConfig`` ↔ ``context:``, ``RunnerConfig`` ↔ ``runner_config:``
…). An instance keeps only the keys that were set, so ``ConfigArguments(...).to_config()`` (or
``Trainer(args=ConfigArguments(...))``) overrides exactly those keys of the task's default configuration. Keys outside
``_support_kwargs`` are rejected with the list of valid names.

Reference: ``mindformers/trainer/config_args.py`` (``BaseArgsConfig:41``, ``ContextConfig:69``,
``ParallelContextConfig:539``, ``ParallelConfig:746``, ``RunnerConfig:798``, ``CheckpointConfig:837``,
``LRConfig:866``, ``OptimizerConfig:885``, ``WrapperConfig:911``, ``DatasetConfig:972``, ``ConfigArguments:1017``).
Keys that only steer the Ascend runtime (graph kernel flags, dump paths, ``ascend_config`` …) are accepted and
carried into the configuration unchanged; nothing on a B200 reads them.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional


class BaseArgsConfig:
    """Base of the dataclass mirrors of the YAML sections (reference ``trainer/config_args.py``): keeps unknown keys,
    drops ``None`` values in ``to_dict``."""

    _support_kwargs: List[str] = []
    _section: Optional[str] = None          # YAML section this class mirrors

    def __init__(self, **kwargs):
        unknown = [k for k in kwargs if k not in self._support_kwargs]
        if unknown:
            raise KeyError(f"{type(self).__name__} does not accept {unknown}; valid keys: {self._support_kwargs}")
        for k, v in kwargs.items():
            if v is None:
                continue
            if isinstance(v, BaseArgsConfig):
                v = v.to_dict()
            elif isinstance(v, (list, tuple)):
                v = [x.to_dict() if isinstance(x, BaseArgsConfig) else x for x in v]
            setattr(self, k, v)

    @classmethod
    def get_supported_kwargs(cls) -> List[str]:
        return list(cls._support_kwargs)

    @classmethod
    def filter_kwargs(cls, **kwargs) -> Dict[str, Any]:
        return {k: v for k, v in kwargs.items() if k in cls._support_kwargs}

    def to_dict(self) -> Dict[str, Any]:
        return {k: v for k, v in vars(self).items() if not k.startswith("_")}

    def __repr__(self):
        return f"{type(self).__name__}({self.to_dict()})"


class ContextConfig(BaseArgsConfig):
    """``context:`` — device, memory limit, determinism and the (ignored here) graph-compiler switches."""
    _section = "context"
    _support_kwargs = [
        "mode", "device_target", "device_id", "max_device_memory", "variable_memory_max_size", "mempool_block_size",
        "op_timeout", "save_graphs", "save_graphs_path", "enable_dump", "save_dump_path", "deterministic",
        "print_file_path", "env_config_path", "precompile_only", "reserve_class_name_in_scope", "pynative_synchronize",
        "enable_graph_kernel", "graph_kernel_flags", "enable_reduce_precision", "check_bprop", "max_call_depth",
        "grad_for_scalar", "enable_compile_cache", "compile_cache_path", "inter_op_parallel_num", "runtime_num_threads",
        "memory_optimize_level", "memory_offload", "ascend_config", "jit_config", "jit_level", "infer_boost",
        "affinity_cpu_list", "exec_order", "jit_syntax_level", "disable_format_transform", "support_binary",
        "gpu_config", "debug_level", "device_type"]


class MFContextConfig(BaseArgsConfig):
    """Top-level run switches that the reference keeps beside ``context``."""
    _section = None
    _support_kwargs = ["local_rank", "device_num", "run_mode", "seed", "output_dir", "load_checkpoint",
                       "src_strategy_path_or_dir", "auto_trans_ckpt", "transform_process_num", "only_save_strategy",
                       "resume_training", "load_ckpt_format", "use_parallel", "use_legacy", "pretrained_model_dir",
                       "train_precision_sync", "infer_precision_sync", "remote_save_url", "profile", "use_graceful_exit"]


class ParallelContextConfig(BaseArgsConfig):
    """``parallel:`` — the automatic-parallel context of the reference; the keys that matter here are
    ``enable_parallel_optimizer`` (distributed optimizer), ``gradients_mean`` and ``strategy_ckpt_config``."""
    _section = "parallel"
    _support_kwargs = [
        "device_num", "global_rank", "gradients_mean", "gradient_fp32_sync", "parallel_mode", "auto_parallel_search_mode",
        "search_mode", "parameter_broadcast", "strategy_ckpt_load_file", "strategy_ckpt_save_file", "full_batch",
        "enable_parallel_optimizer", "enable_alltoall", "all_reduce_fusion_config", "pipeline_stages",
        "pipeline_result_broadcast", "grad_accumulation_step", "parallel_optimizer_config", "comm_fusion",
        "strategy_ckpt_config", "dataset_strategy", "full_batch_strategy"]


class ParallelConfig(BaseArgsConfig):
    """``parallel_config:`` — the degrees of every parallel axis."""
    _section = "parallel_config"
    _support_kwargs = [
        "data_parallel", "model_parallel", "context_parallel", "expert_parallel", "pipeline_stage", "micro_batch_num",
        "seq_split_num", "use_seq_parallel", "optimizer_shard", "gradient_aggregation_group", "vocab_emb_dp",
        "context_parallel_algo", "ulysses_degree_in_cp", "mem_coeff", "expert_model_parallel", "recompute",
        "micro_batch_interleave_num", "virtual_pipeline_stage"]


class CloudConfig(BaseArgsConfig):
    """Object-storage sync of outputs (a local directory plays the remote here)."""
    _section = None
    _support_kwargs = ["obs_path", "root_path", "rank_id", "upload_frequence", "keep_last", "retry", "retry_time",
                       "remote_save_url"]


class RunnerConfig(BaseArgsConfig):
    """``runner_config:``"""
    _section = "runner_config"
    _support_kwargs = ["epochs", "batch_size", "sink_mode", "sink_size", "initial_epoch", "has_trained_epoches",
                       "has_trained_steps", "image_size", "num_classes", "gradient_accumulation_steps",
                       "stop_step", "max_steps"]


class CheckpointConfig(BaseArgsConfig):
    """The ``CheckpointMonitor`` entry of ``callbacks:``."""
    _section = "callbacks"
    _support_kwargs = ["prefix", "directory", "config", "save_checkpoint_steps", "save_checkpoint_seconds",
                       "keep_checkpoint_max", "keep_checkpoint_per_n_minutes", "integrated_save", "save_network_params",
                       "save_trainable_params", "async_save", "saved_network", "append_info", "enc_key", "enc_mode",
                       "exception_save", "global_batch_size", "checkpoint_format", "remove_redundancy",
                       "embedding_size", "embedding_local_norm_threshold", "use_checkpoint_health_monitor",
                       "health_ckpts_record_dir"]

    def to_dict(self):
        d = super().to_dict()
        d["type"] = "CheckpointMonitor"
        return d


class LRConfig(BaseArgsConfig):
    """``lr_schedule:`` — ``lr_type`` names the schedule class; other keys go to its constructor."""
    _section = "lr_schedule"
    _support_kwargs = ["type", "learning_rate", "lr_end", "warmup_steps", "warmup_ratio", "warmup_lr_init",
                       "total_steps", "decay_steps", "decay_ratio", "power", "num_cycles", "lr_end1", "lr_end2",
                       "decay_rate", "min_lr", "max_lr", "cycle", "stable_steps"]

    def __init__(self, lr_type: Optional[str] = None, **kwargs):
        if lr_type is not None:
            kwargs["type"] = lr_type
        super().__init__(**kwargs)


class OptimizerConfig(BaseArgsConfig):
    """``optimizer:`` — ``optim_type`` names the optimizer class."""
    _section = "optimizer"
    _support_kwargs = ["type", "learning_rate", "beta1", "beta2", "betas", "eps", "weight_decay", "use_nesterov",
                       "momentum", "loss_scale", "params", "swap", "fused_num", "interleave_step"]

    def __init__(self, optim_type: Optional[str] = None, learning_rate=None, **kwargs):
        if optim_type is not None:
            kwargs["type"] = optim_type
        if learning_rate is not None:
            kwargs["learning_rate"] = learning_rate
        super().__init__(**kwargs)


class WrapperConfig(BaseArgsConfig):
    """``runner_wrapper:`` — the train-step wrapper and its loss-scale manager."""
    _section = "runner_wrapper"
    _support_kwargs = ["type", "sens", "scale_sense", "use_clip_grad", "max_grad_norm", "local_norm", "calculate_per_token_loss"]

    def __init__(self, wrapper_type: Optional[str] = None, **kwargs):
        if wrapper_type is not None:
            kwargs["type"] = wrapper_type
        super().__init__(**kwargs)


class DataLoaderConfig(BaseArgsConfig):
    """The ``data_loader`` entry of a dataset section."""
    _section = None
    _support_kwargs = ["type", "dataset_dir", "dataset_files", "num_samples", "num_parallel_workers", "shuffle",
                       "sampler", "extensions", "class_indexing", "language_pair", "decode", "num_shards", "shard_id",
                       "cache", "decrypt", "task", "usage", "stage", "column_names", "anno_path", "tokenizer",
                       "dataset_name", "file_format", "max_length", "phase", "origin_columns", "path", "split",
                       "handler", "sizes", "datasets_type", "config", "path_prefix", "seq_length"]

    def __init__(self, dataloader_type: Optional[str] = None, **kwargs):
        if dataloader_type is not None:
            kwargs["type"] = dataloader_type
        super().__init__(**kwargs)


class DatasetConfig(BaseArgsConfig):
    """``train_dataset`` / ``eval_dataset``."""
    _section = "train_dataset"
    _support_kwargs = ["data_loader", "input_columns", "output_columns", "column_order", "drop_remainder", "repeat",
                       "batch_size", "image_size", "num_parallel_workers", "python_multiprocessing", "numa_enable",
                       "prefetch_size", "seed", "tokenizer", "max_seq_length", "max_source_length", "max_target_length",
                       "ignore_pad_token_for_loss", "phase", "eod_reset", "eod_token_id", "pad_token_id",
                       "dynamic_batch", "divisor", "remainder", "shuffle", "pin_memory", "construct_args_key"]


class ConfigArguments(BaseArgsConfig):
    """The whole run: sections as objects (or dicts) plus top-level switches. ``to_config()`` gives the nested dict
    that ``MindFormerConfig.merge_from_dict`` / ``Trainer(args=…)`` take."""
    _support_kwargs = ["output_dir", "profile", "auto_tune", "filepath_prefix", "autotune_per_step", "seed",
                       "train_dataset", "eval_dataset", "runner_config", "optimizer", "lr_schedule", "runner_wrapper",
                       "save_checkpoint", "cloud_config", "context", "parallel", "parallel_config", "use_parallel",
                       "run_mode", "load_checkpoint", "resume_training", "auto_trans_ckpt", "only_save_strategy",
                       "src_strategy_path_or_dir", "callbacks", "eval_callbacks", "do_eval", "eval_step_interval",
                       "eval_epoch_interval", "micro_batch_interleave_num", "recompute_config"]

    def __init__(self, output_dir: Optional[str] = None, profile: Optional[bool] = None, seed: Optional[int] = None,
                 train_dataset=None, eval_dataset=None, runner_config=None, optimizer=None, lr_schedule=None,
                 runner_wrapper=None, save_checkpoint=None, context=None, parallel=None, parallel_config=None,
                 **kwargs):
        super().__init__(output_dir=output_dir, profile=profile, seed=seed, train_dataset=train_dataset,
                         eval_dataset=eval_dataset, runner_config=runner_config, optimizer=optimizer,
                         lr_schedule=lr_schedule, runner_wrapper=runner_wrapper, save_checkpoint=save_checkpoint,
                         context=context, parallel=parallel, parallel_config=parallel_config, **kwargs)

    def to_config(self) -> Dict[str, Any]:
        cfg = self.to_dict()
        ckpt = cfg.pop("save_checkpoint", None)
        if ckpt is not None:
            cbs = [c for c in (cfg.get("callbacks") or []) if c.get("type") != "CheckpointMonitor"]
            cfg["callbacks"] = cbs + [ckpt]
        for key in ("train_dataset", "eval_dataset"):
            ds = cfg.get(key)
            if ds is not None:
                cfg[key + "_task"] = {"type": "CausalLanguageModelDataset", "dataset_config": ds}
        return cfg
