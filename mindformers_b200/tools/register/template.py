"""Schema and defaults of the top-level YAML sections.

Plays the role of the reference's ``mindformers/tools/register/template.py`` (sections at
:235-560, ``ConfigTemplate.apply_template`` :639-662): general keys live at the top level of the
YAML, every other section is a mapping with defaults; strict sections reject unknown keys; the
set of sections kept depends on ``run_mode``; ``moe_config`` is dropped for the Megatron-style
stack (``use_legacy: False``, :682-683). Defaults that name Ascend (``device_target``) are replaced
by their CUDA counterparts.
"""
from __future__ import annotations

import copy
import logging
from typing import Dict, List

logger = logging.getLogger("mindformers_b200")

GENERAL_DEFAULTS = dict(
    seed=1, output_dir="./output", run_mode=None, use_parallel=False, resume_training=False,
    load_checkpoint="", load_ckpt_format="safetensors", auto_trans_ckpt=False, transform_process_num=1,
    src_strategy_path_or_dir="", only_save_strategy=False, load_ckpt_async=False, use_legacy=True,
    pretrained_model_dir="", do_eval=False, eval_step_interval=100, eval_epoch_interval=-1,
    ignore_data_skip=False, data_skip_steps=None, profile=False, profile_communication=False,
    profile_memory=True, init_start_profile=False, profile_start_step=1, profile_stop_step=10,
    profile_rank_ids=None, profile_pipeline=False, profile_level=1, mstx=False, layer_scale=False,
    layer_decay=0.65, lr_scale=False, lr_scale_factor=256, micro_batch_interleave_num=1,
    remote_save_url=None, save_file=None, input_data=None, predict_batch_size=None, adapter_id=None,
    exclude_cann_cpu=False, train_precision_sync=None, infer_precision_sync=None,
    postprocess_use_numpy=False, remove_redundancy=False, use_graceful_exit=False,
)

SECTION_DEFAULTS: Dict[str, dict] = {
    "parallel_config": dict(
        data_parallel=1, model_parallel=1, context_parallel=1, expert_parallel=1, pipeline_stage=1,
        micro_batch_num=1, seq_split_num=1, use_seq_parallel=False, optimizer_shard=None,
        gradient_aggregation_group=4, vocab_emb_dp=True, context_parallel_algo="colossalai_cp",
        ulysses_degree_in_cp=1, mem_coeff=0.1, pp_interleave_num=1, expert_model_parallel=None),
    "recompute_config": dict(
        recompute=False, select_recompute=False, parallel_optimizer_comm_recompute=False,
        select_comm_recompute=False, mp_comm_recompute=True, recompute_slice_activation=False,
        select_recompute_exclude=False, select_comm_recompute_exclude=False),
    "swap_config": dict(swap=False, layer_swap=None, op_swap=None, default_prefetch=1),
    "moe_config": dict(
        expert_num=1, capacity_factor=1.1, aux_loss_factor=0.05, num_experts_chosen=1,
        expert_group_size=None, group_wise_a2a=False, comp_comm_parallel=False,
        comp_comm_parallel_degree=2, save_token_distribution=False, cur_layer=0,
        enable_cold_hot_expert=False, update_step=10000, hot_expert_num=0, cold_token_percent=1.0,
        moe_module_name="", routing_policy="TopkRouterV1", norm_topk_prob=True, enable_sdrop=False,
        use_fused_ops_topkrouter=False, router_dense_type="float32", shared_expert_num=0,
        use_shared_expert_gating=False, max_router_load=128 * 1024, topk_method="greedy", topk_group=None,
        n_group=None, first_k_dense_replace=True, moe_intermediate_size=1407, routed_scaling_factor=1.0,
        aux_loss_types=None, aux_loss_factors=None, z_loss_factor=0.0, balance_via_topk_bias=False,
        topk_bias_update_rate=0.0, use_allgather_dispatcher=False, moe_shared_expert_overlap=False,
        expert_model_parallel=None, use_gating_sigmoid=False, enable_deredundency=False,
        npu_nums_per_device=1, use_gmm=False, enable_gmm_safe_tokens=False, use_fused_ops_permute=False,
        callback_moe_droprate=False, dispatch_global_max_bs=0, ep_extend_tp=True),
    "runner_config": dict(batch_size=1, epochs=1, sink_mode=1, sink_size=1, gradient_accumulation_steps=1,
                          num_classes=1, stop_step=0),
    "parallel": dict(parallel_mode=1, full_batch=True, search_mode="sharding_propagation",
                     enable_parallel_optimizer=False, gradients_mean=False, enable_alltoall=False,
                     strategy_ckpt_save_file="./ckpt_strategy.ckpt"),
    "context": dict(mode=0, device_target="CUDA", device_id=0, max_device_memory="170GB",
                    max_call_depth=10000),
    "train_dataset": {}, "train_dataset_task": {}, "processor": {}, "eval_dataset": {},
    "eval_dataset_task": {}, "trainer": {}, "model": {},
    "runner_wrapper": dict(type="MFTrainOneStepCell", use_clip_grad=True,
                           scale_sense=dict(type="DynamicLossScaleUpdateCell", loss_scale_value=65536,
                                            scale_factor=2, scale_window=1000)),
    "optimizer": dict(type="AdamW", betas=[0.9, 0.999], learning_rate=5.0e-5, eps=1.0e-8, weight_decay=0.0),
    "lr_schedule": dict(type="CosineWithWarmUpLR", learning_rate=5.0e-5, lr_end=0.0, warmup_ratio=0.0,
                        total_steps=-1),
    "metric": dict(type="PerplexityMetric"),
    "callbacks": [dict(type="MFLossMonitor")],
    "eval_callbacks": [],
    "monitor_config": dict(
        monitor_on=False, dump_path="", target=None, invert=False, step_interval=1, local_loss_format=None,
        local_norm_format=None, device_local_norm_format=None, device_local_loss_format=None,
        optimizer_state_format=None, weight_state_format=None, throughput_baseline=None,
        print_struct=False, check_for_global_norm=False, global_norm_spike_threshold=3.0,
        global_norm_spike_count_threshold=10),
    "tensorboard": {},
}

# sections whose keys are checked against the defaults
STRICT_SECTIONS = {"parallel_config", "recompute_config", "swap_config", "moe_config", "runner_config",
                   "monitor_config"}
# sections that must name a ``type`` when present
TYPED_SECTIONS = {"train_dataset_task", "eval_dataset_task", "trainer", "runner_wrapper", "optimizer",
                  "lr_schedule", "metric"}
# "spec" sections: when the user changes ``type`` the defaults of the default type do not apply
SPEC_SECTIONS = {"runner_wrapper", "optimizer", "lr_schedule", "metric"}

GENERAL_SECTIONS = ["context", "parallel", "trainer", "model", "moe_config", "parallel_config",
                    "recompute_config", "swap_config", "monitor_config", "tensorboard"]
TRAIN_SECTIONS = ["runner_config", "train_dataset", "train_dataset_task", "runner_wrapper", "optimizer",
                  "lr_schedule", "callbacks"]
DO_EVAL_SECTIONS = ["eval_dataset", "eval_dataset_task", "eval_callbacks", "metric"]
PREDICT_SECTIONS = ["processor", "runner_config"]
EVAL_SECTIONS = ["runner_config", "eval_dataset", "eval_dataset_task", "eval_callbacks", "metric"]
RUN_MODES = ("train", "finetune", "eval", "predict")


class ConfigTemplate:
    """Fill defaults, validate keys and drop sections that the run mode does not use."""

    @staticmethod
    def sections_for(run_mode, do_eval=False) -> List[str]:
        if run_mode in ("train", "finetune"):
            names = GENERAL_SECTIONS + TRAIN_SECTIONS + (DO_EVAL_SECTIONS if do_eval else [])
        elif run_mode == "predict":
            names = GENERAL_SECTIONS + PREDICT_SECTIONS
        elif run_mode == "eval":
            names = GENERAL_SECTIONS + EVAL_SECTIONS
        else:
            if run_mode is not None:
                logger.warning("run_mode %r is not one of %s; only the general sections are kept",
                               run_mode, RUN_MODES)
            names = list(GENERAL_SECTIONS)
        seen, out = set(), []
        for n in names:
            if n not in seen:
                seen.add(n)
                out.append(n)
        return out

    @classmethod
    def apply_template(cls, config: dict):
        """In-place normalisation of a configuration mapping."""
        use_legacy = config.get("use_legacy", True)
        run_mode = config.get("run_mode")
        for key, default in GENERAL_DEFAULTS.items():
            config.setdefault(key, copy.deepcopy(default))
        keep = cls.sections_for(run_mode, bool(config.get("do_eval")))
        for name in keep:
            if name == "moe_config" and not use_legacy:
                config.pop(name, None)
                continue
            config[name] = cls._apply_section(name, config.get(name))
        known = set(GENERAL_DEFAULTS) | set(keep)
        unused = [k for k in list(config) if k not in known and k in SECTION_DEFAULTS]
        for k in unused:
            config.pop(k)
        if unused:
            logger.warning("sections %s are not used in run_mode %r and were dropped", unused, run_mode)
        return config

    @staticmethod
    def _apply_section(name: str, given):
        default = SECTION_DEFAULTS[name]
        if isinstance(default, list):
            if given is None:
                return copy.deepcopy(default)
            if not isinstance(given, (list, tuple)):
                raise ValueError(f"section {name!r} must be a list of mappings")
            for item in given:
                if not isinstance(item, dict) or "type" not in item:
                    raise ValueError(f"every entry of {name!r} needs a 'type'")
            return list(given)
        if given is None:
            return copy.deepcopy(default)
        if not isinstance(given, dict):
            raise ValueError(f"section {name!r} must be a mapping, got {type(given).__name__}")
        if name in STRICT_SECTIONS:
            unknown = sorted(set(given) - set(default))
            if unknown:
                raise KeyError(f"unknown key(s) {unknown} in section {name!r}")
        if name in TYPED_SECTIONS and given and "type" not in given and "type" not in default:
            raise KeyError(f"section {name!r} needs a 'type'")
        if name in SPEC_SECTIONS and given.get("type", default.get("type")) != default.get("type"):
            return copy.deepcopy(dict(given))
        merged = copy.deepcopy(default)
        for k, v in given.items():
            if isinstance(v, dict) and isinstance(merged.get(k), dict) and name not in SPEC_SECTIONS:
                merged[k].update(v)
            else:
                merged[k] = v
        return merged
