"""Named architecture presets (HF-style key/value dictionaries) for the shipped model families.

These are the shapes of the public model cards; they feed ``convert_to_transformer_config`` exactly as
a ``config.json`` of the same model would.
"""
from __future__ import annotations

import copy

PRESETS = {
    "llama3_1_8b": dict(
        model_type="llama", num_hidden_layers=32, hidden_size=4096, num_attention_heads=32,
        num_key_value_heads=8, intermediate_size=14336, vocab_size=128256, rms_norm_eps=1e-5,
        rope_theta=500000.0, max_position_embeddings=131072, tie_word_embeddings=False,
        rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                          original_max_position_embeddings=8192)),
    "llama3_1_70b": dict(
        model_type="llama", num_hidden_layers=80, hidden_size=8192, num_attention_heads=64,
        num_key_value_heads=8, intermediate_size=28672, vocab_size=128256, rms_norm_eps=1e-5,
        rope_theta=500000.0, max_position_embeddings=131072, tie_word_embeddings=False,
        rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                          original_max_position_embeddings=8192)),
    "llama2_7b": dict(
        model_type="llama", num_hidden_layers=32, hidden_size=4096, num_attention_heads=32,
        num_key_value_heads=32, intermediate_size=11008, vocab_size=32000, rms_norm_eps=1e-5,
        rope_theta=10000.0, max_position_embeddings=4096),
    "qwen2_5_7b": dict(
        model_type="qwen2", num_hidden_layers=28, hidden_size=3584, num_attention_heads=28,
        num_key_value_heads=4, intermediate_size=18944, vocab_size=152064, rms_norm_eps=1e-6,
        rope_theta=1000000.0, max_position_embeddings=131072, attention_bias=True, tie_word_embeddings=False),
    "qwen3_8b": dict(
        model_type="qwen3", num_hidden_layers=36, hidden_size=4096, num_attention_heads=32,
        num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=151936, rms_norm_eps=1e-6,
        rope_theta=1000000.0, max_position_embeddings=40960, qk_layernorm=True, tie_word_embeddings=False),
    "qwen3_32b": dict(
        model_type="qwen3", num_hidden_layers=64, hidden_size=5120, num_attention_heads=64,
        num_key_value_heads=8, head_dim=128, intermediate_size=25600, vocab_size=151936, rms_norm_eps=1e-6,
        rope_theta=1000000.0, max_position_embeddings=40960, qk_layernorm=True, tie_word_embeddings=False),
    "qwen3_30b_a3b": dict(
        model_type="qwen3_moe", num_hidden_layers=48, hidden_size=2048, num_attention_heads=32,
        num_key_value_heads=4, head_dim=128, intermediate_size=6144, moe_intermediate_size=768,
        num_experts=128, num_experts_per_tok=8, norm_topk_prob=True, vocab_size=151936, rms_norm_eps=1e-6,
        rope_theta=1000000.0, max_position_embeddings=40960, qk_layernorm=True, tie_word_embeddings=False,
        first_k_dense_replace=0, moe_router_score_function="softmax", router_aux_loss_coef=1e-3),
    "deepseek_v3": dict(
        model_type="deepseek_v3", num_hidden_layers=61, hidden_size=7168, num_attention_heads=128,
        num_key_value_heads=128, intermediate_size=18432, moe_intermediate_size=2048, n_routed_experts=256,
        n_shared_experts=1, num_experts_per_tok=8, n_group=8, topk_group=4, routed_scaling_factor=2.5,
        norm_topk_prob=True, scoring_func="sigmoid", first_k_dense_replace=3, vocab_size=129280,
        rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=163840, q_lora_rank=1536,
        kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
        num_nextn_predict_layers=1, moe_router_enable_expert_bias=True, tie_word_embeddings=False,
        rope_interleave=True,
        rope_scaling=dict(type="yarn", factor=40.0, beta_fast=32.0, beta_slow=1.0, mscale=1.0, mscale_all_dim=1.0,
                          original_max_position_embeddings=4096)),
    "tiny_llama": dict(
        model_type="llama", num_hidden_layers=2, hidden_size=256, num_attention_heads=4, num_key_value_heads=2,
        intermediate_size=688, vocab_size=1024, rms_norm_eps=1e-5, rope_theta=10000.0,
        max_position_embeddings=128),
}


def get_preset(name: str, **overrides) -> dict:
    if name not in PRESETS:
        raise KeyError(f"unknown preset {name!r}; known: {sorted(PRESETS)}")
    cfg = copy.deepcopy(PRESETS[name])
    cfg.update(overrides)
    return cfg


def preset_is_mla(cfg: dict) -> bool:
    return "kv_lora_rank" in cfg
