"""Translate HF-style / YAML-style model configuration keys into ``TransformerConfig`` fields.

Behavioural counterpart of the reference's ``parallel_core/transformer_config_utils.py``
(``COMMON_CONFIG_MAPPING`` :202-421, ``convert_to_transformer_config`` :424-506): each target field
lists the aliases it accepts; two aliases of one field given together are an error; keys that map
to nothing raise unless white-listed.
"""
from __future__ import annotations

import dataclasses
from typing import Optional, Union

from .transformer_config import MLATransformerConfig, TransformerConfig


def _is_fp32(v):
    return str(v).lower().replace("torch.", "") in ("float32", "fp32", "float")


def _score_fn(v):
    if isinstance(v, bool):
        return "sigmoid" if v else "softmax"
    return str(v)


def _drop_policy(v):
    if isinstance(v, bool):
        return "position" if v else "probs"
    return v


def _cp_comm(v):
    return {"colossalai_cp": "all_gather", "ulysses_cp": "a2a", "hybrid_cp": "a2a+p2p"}.get(v, v)


def _recompute(v):
    return v


# target field -> (aliases, optional transform)
_TABLE = [
    ("data_parallel_size", ("data_parallel", "data_parallel_size"), None),
    ("tensor_model_parallel_size", ("model_parallel", "tensor_model_parallel_size"), None),
    ("pipeline_model_parallel_size", ("pipeline_stage", "pipeline_model_parallel_size"), None),
    ("virtual_pipeline_model_parallel_size", ("pp_interleave_num", "virtual_pipeline_model_parallel_size"), None),
    ("sequence_parallel", ("use_seq_parallel", "sequence_parallel"), None),
    ("context_parallel_size", ("context_parallel", "context_parallel_size"), None),
    ("expert_model_parallel_size", ("expert_parallel", "expert_model_parallel_size"), None),
    ("expert_tensor_parallel_size", ("expert_model_parallel", "expert_tensor_parallel_size"), None),
    ("params_dtype", ("param_init_type", "params_dtype"), None),
    ("cpu_offloading", ("swap", "cpu_offloading"), None),
    ("cpu_offloading_num_layers", ("layer_swap", "cpu_offloading_num_layers"), None),
    ("mtp_num_layers", ("mtp_depth", "num_nextn_predict_layers", "mtp_num_layers"), None),
    ("mtp_loss_scaling_factor", ("mtp_loss_factor", "mtp_loss_scaling_factor"), None),
    ("num_attention_heads", ("num_heads", "num_attention_heads"), None),
    ("num_query_groups", ("n_kv_heads", "num_key_value_heads", "multi_query_group_num", "num_query_groups"), None),
    ("vocab_size", ("padded_vocab_size", "vocab_size"), None),
    ("ffn_hidden_size", ("intermediate_size", "ffn_hidden_size"), None),
    ("kv_channels", ("head_dim", "kv_channels"), None),
    ("fp32_residual_connection", ("fp32_residual_connection",), None),
    ("residual_dtype", ("residual_dtype",), None),
    ("layernorm_epsilon", ("rms_norm_eps", "layernorm_epsilon"), None),
    ("add_qkv_bias", ("qkv_has_bias", "attention_bias", "add_qkv_bias"), None),
    ("num_moe_experts", ("expert_num", "n_routed_experts", "num_experts", "num_moe_experts"), None),
    ("num_layers", ("num_layers", "num_hidden_layers"), None),
    ("rotary_interleaved", ("rope_interleave", "rotary_interleaved"), None),
    ("position_embedding_type", ("extend_method", "position_embedding_type"), None),
    ("init_method_std", ("init_method_std", "initializer_range"), None),
    ("attention_softmax_in_fp32", ("attention_softmax_in_fp32",), None),
    ("softmax_compute_dtype", ("softmax_compute_dtype",), None),
    ("apply_rope_fusion", ("use_fused_rope", "apply_rope_fusion"), None),
    ("bias_swiglu_fusion", ("use_fused_swiglu", "bias_swiglu_fusion"), None),
    ("recompute", ("recompute",), _recompute),
    ("moe_ffn_hidden_size", ("moe_intermediate_size", "moe_ffn_hidden_size"), None),
    ("moe_router_topk", ("num_experts_chosen", "num_experts_per_tok", "moe_router_topk"), None),
    ("moe_router_num_groups", ("n_group", "moe_router_num_groups"), None),
    ("moe_router_group_topk", ("topk_group", "moe_router_group_topk"), None),
    ("moe_router_topk_scaling_factor", ("routed_scaling_factor", "moe_router_topk_scaling_factor"), None),
    ("moe_router_score_function", ("use_gating_sigmoid", "scoring_func", "moe_router_score_function"), _score_fn),
    ("moe_router_dtype", ("router_dense_type", "moe_router_dtype"), None),
    ("moe_router_enable_expert_bias", ("balance_via_topk_bias", "moe_router_enable_expert_bias"), None),
    ("moe_router_bias_update_rate", ("topk_bias_update_rate", "moe_router_bias_update_rate"), None),
    ("moe_grouped_gemm", ("use_gmm", "moe_grouped_gemm"), None),
    ("moe_z_loss_coeff", ("z_loss_factor", "moe_z_loss_coeff"), None),
    ("moe_aux_loss_coeff", ("router_aux_loss_coef", "moe_aux_loss_coeff"), None),
    ("moe_expert_capacity_factor", ("capacity_factor", "moe_expert_capacity_factor"), None),
    ("moe_token_drop_policy", ("enable_sdrop", "moe_token_drop_policy"), _drop_policy),
    ("use_pad_tokens", ("enable_gmm_safe_tokens", "use_pad_tokens"), None),
    ("shared_expert_num", ("n_shared_experts", "shared_expert_num"), None),
    ("moe_shared_expert_intermediate_size", ("shared_expert_intermediate_size", "moe_shared_expert_intermediate_size"), None),
    ("use_shared_expert_gating", ("use_shared_expert_gating",), None),
    ("cp_comm_type", ("cp_comm_type",), None),
    ("context_parallel_algo", ("context_parallel_algo",), None),
    ("hierarchical_context_parallel_sizes", ("hierarchical_context_parallel_sizes",), None),
    ("ulysses_degree_in_cp", ("ulysses_degree_in_cp",), None),
    ("qk_head_dim", ("qk_nope_head_dim", "qk_head_dim"), None),
    ("qk_pos_emb_head_dim", ("qk_rope_head_dim", "qk_pos_emb_head_dim"), None),
    ("rotary_base", ("theta", "rope_theta", "rotary_base"), None),
    ("rotary_percent", ("partial_rotary_factor", "rotary_percent"), None),
    ("rotary_scaling_factor", ("scaling_factor", "factor", "rotary_scaling_factor"), None),
    ("max_position_embeddings", ("max_position_embeddings",), None),
    ("original_max_position_embeddings", ("original_max_position_embeddings",), None),
]

_MAPPED_TARGETS = {t for t, _, _ in _TABLE}
_ALIAS: dict = {}
for _target, _aliases, _fn in _TABLE:
    for _a in _aliases:
        _ALIAS[_a] = (_target, _fn)

# keys that a model configuration may carry without a TransformerConfig counterpart
DEFAULT_WHITE_KEYS = {
    # resolved into model_parallel / context_parallel before the model is built (core/context.py)
    "use_3d_tensor_parallel", "tp_x", "tp_y", "tp_z",
    "model_type", "architectures", "type", "torch_dtype", "dtype", "transformers_version", "auto_map",
    "bos_token_id", "eos_token_id", "use_cache", "use_sliding_window", "sliding_window",
    "max_window_layers", "attention_bias_", "pretraining_tp", "mlp_bias", "monitor_config",
    "dataset_config", "batch_size", "multiple_of", "ffn_dim_multiplier", "qkv_concat", "use_past",
    "input_sliced_sig", "return_extra_loss", "moe_config", "checkpoint_name_or_path", "name_or_path",
    "_name_or_path", "tokenizer_class", "top_k", "top_p", "do_sample", "repetition_penalty",
    "max_decode_length", "max_length", "temperature", "output_router_logits", "decoder_sparse_step",
    "mlp_only_layers", "ep_size", "num_nextn_predict_layers_", "quantization_config", "layer_types",
    "rope_parameters", "is_encoder_decoder", "generation_config", "return_dict", "output_attentions",
    "output_hidden_states", "id2label", "label2id", "problem_type", "chunk_size_feed_forward",
    "tie_encoder_decoder", "add_cross_attention", "is_decoder", "cross_attention_hidden_size",
    "prefix", "finetuning_task", "task_specific_params", "tf_legacy_loss", "torchscript",
    "pruned_heads", "sep_token_id", "decoder_start_token_id", "_attn_implementation_autoset",
    "attn_implementation", "_attn_implementation", "use_bfloat16", "tokenizer",
    # ChatGLM / GLM-4 keys that the family's configuration class folds into other fields
    "rmsnorm", "post_layer_norm", "multi_query_attention", "apply_query_key_layer_scaling", "rope_ratio",
    "bias_dropout_fusion", "apply_residual_connection_post_layernorm", "original_rope", "classifier_dropout",
    "mlp_concat", "use_rearrange_rope", "quantization_bit", "pre_seq_len", "prefix_projection", "gmask_token_id",
}

_FIELDS = {f.name for f in dataclasses.fields(MLATransformerConfig)}


def convert_to_transformer_config(model_config, is_mla_model: bool = False, additional_map: Optional[dict] = None,
                                  not_convert_whitelist: Optional[set] = None,
                                  strict: bool = True) -> Union[TransformerConfig, MLATransformerConfig]:
    """Build a ``TransformerConfig`` (``MLATransformerConfig`` for MLA models) from a model config.

    ``model_config`` is a mapping or an object with ``to_dict()``; its optional ``parallel_config``
    sub-mapping contributes the parallel sizes. ``additional_map`` adds ``{alias: field}`` entries.
    """
    if model_config is None:
        raise ValueError("model_config is required")
    if hasattr(model_config, "to_dict") and not isinstance(model_config, dict):
        model_config = model_config.to_dict()
    if not isinstance(model_config, dict):
        raise ValueError(f"model_config must be a mapping, got {type(model_config).__name__}")
    model_config = dict(model_config)
    alias = dict(_ALIAS)
    for k, v in (additional_map or {}).items():
        alias[k] = v if isinstance(v, tuple) else (v, None)
    white = set(DEFAULT_WHITE_KEYS) | set(not_convert_whitelist or ())

    out: dict = {}
    origin: dict = {}

    def put(key, value):
        if key in alias:
            target, fn = alias[key]
        elif key in _FIELDS:
            target, fn = key, None
        else:
            return False
        if target in out and origin[target] != key:
            raise KeyError(f"conflicting settings for {target!r}: {origin[target]!r} and {key!r}")
        out[target] = fn(value) if fn else value
        origin[target] = key
        return True

    parallel = model_config.pop("parallel_config", None)
    if parallel is not None:
        if hasattr(parallel, "to_dict") and not isinstance(parallel, dict):
            parallel = parallel.to_dict()
        for k, v in dict(parallel).items():
            put(k, v)
    unknown = []
    for k, v in model_config.items():
        if k in white:
            continue
        if v is None and k not in _FIELDS:
            continue
        if not put(k, v):
            unknown.append(k)
    if unknown and strict:
        raise ValueError(f"configuration keys {unknown} have no TransformerConfig counterpart")

    # derived values with HF semantics
    rs = out.get("rope_scaling")
    if isinstance(rs, dict):
        rtype = rs.get("rope_type", rs.get("type"))
        if rtype == "llama3":
            out.setdefault("use_rope_scaling", True)
            out.setdefault("rope_type", "llama3")
        elif rtype == "yarn":
            out.setdefault("rope_type", "yarn")
            for src, dst in (("factor", "rotary_scaling_factor"), ("beta_fast", "beta_fast"),
                             ("beta_slow", "beta_slow"), ("mscale", "mscale"),
                             ("mscale_all_dim", "mscale_all_dim"),
                             ("original_max_position_embeddings", "original_max_position_embeddings")):
                if src in rs:
                    out[dst] = rs[src]
    if out.get("residual_dtype") is not None and _is_fp32(out["residual_dtype"]):
        out.setdefault("fp32_residual_connection", True)
    if "softmax_compute_dtype" in out:
        out.setdefault("attention_softmax_in_fp32", _is_fp32(out["softmax_compute_dtype"]))
    if is_mla_model and out.get("rope_type") is None and not isinstance(rs, dict):
        out["rope_type"] = "rope"
    cls = MLATransformerConfig if is_mla_model else TransformerConfig
    valid = {f.name for f in dataclasses.fields(cls)}
    return cls(**{k: v for k, v in out.items() if k in valid})
