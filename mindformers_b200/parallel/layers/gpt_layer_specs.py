"""Layer specs of the GPT family: which classes make up a transformer layer, a decoder stack and an MTP block.

Reference: ``training_graph/base_models/gpt/gpt_layer_specs.py`` (``get_gpt_layer_local_spec`` with its
``num_experts / moe_grouped_gemm / qk_layernorm / multi_latent_attention`` switches, ``get_gpt_decoder_block_spec``
:154-217 with the dense / MoE pattern from ``first_k_dense_replace`` or ``moe_layer_freq``,
``get_gpt_mtp_block_spec``) and ``moe_module_specs.py``. One implementation serves training and inference here, so
one set of specs does too: a model variant changes a spec entry (for instance a different attention class), not the
layer code. ``TransformerLayer`` and ``TransformerBlock`` build themselves from these specs.
"""
from __future__ import annotations

from typing import List, Optional

from ..spec_utils import ModuleSpec
from .attention import CrossAttention, MLASelfAttention, MLASelfAttentionMegatron, SelfAttention
from .mlp import MLP
from .moe import GroupedMLP, MoELayer, SharedExpertMLP, TopKRouter
from .mtp import MultiTokenPredictionBlock, MultiTokenPredictionLayer
from .norm import build_norm
from .transformer_layer import TransformerLayer, TransformerLayerSubmodules


def get_moe_module_spec(num_experts: Optional[int] = None, moe_grouped_gemm: bool = True) -> ModuleSpec:
    """Spec of the MoE sub-layer (router + grouped experts + optional shared experts). Experts are always the
    grouped-GEMM implementation; ``moe_grouped_gemm=False`` is accepted and means the same module."""
    if not num_experts:
        raise ValueError("an MoE spec needs num_experts")
    return ModuleSpec(module=MoELayer, submodules={"router": TopKRouter, "experts": GroupedMLP,
                                                   "shared_experts": SharedExpertMLP})


def get_mlp_module_spec(num_experts: Optional[int] = None, moe_grouped_gemm: bool = True) -> ModuleSpec:
    """Dense gated MLP, or the MoE sub-layer when ``num_experts`` is given."""
    return get_moe_module_spec(num_experts, moe_grouped_gemm) if num_experts else ModuleSpec(module=MLP)


def get_gpt_layer_local_spec(num_experts: Optional[int] = None, moe_grouped_gemm: bool = True,
                             qk_layernorm: bool = False, multi_latent_attention: bool = False,
                             sandwich_norm: bool = False, use_contiguous_weight_layout: bool = True,
                             mla_qkv_concat: bool = True) -> ModuleSpec:
    """Spec of one pre-LN transformer layer.

    ``qk_layernorm`` and the ``[Q|K|V]`` row layout live in the configuration that the attention reads, so those two
    switches select nothing here. ``mla_qkv_concat=False`` selects the multi-latent attention with one module per
    projection (``linear_q_down_proj`` / ``linear_q_up_proj`` / ``linear_kv_down_proj`` / ``linear_kv_up_proj``)
    instead of the concatenated down-projection."""
    norm = ModuleSpec(module=build_norm)
    mla = MLASelfAttention if mla_qkv_concat else MLASelfAttentionMegatron
    attn = ModuleSpec(module=mla if multi_latent_attention else SelfAttention)
    return ModuleSpec(module=TransformerLayer, submodules=TransformerLayerSubmodules(
        input_layernorm=norm, self_attention=attn, pre_mlp_layernorm=norm,
        mlp=get_mlp_module_spec(num_experts, moe_grouped_gemm),
        post_attn_layernorm=norm if sandwich_norm else None, post_mlp_layernorm=norm if sandwich_norm else None))


def get_gpt_layer_spec_for_config(config, is_moe: bool) -> ModuleSpec:
    """``get_gpt_layer_local_spec`` with the switches taken from a ``TransformerConfig``."""
    return get_gpt_layer_local_spec(
        num_experts=config.num_moe_experts if is_moe else None, moe_grouped_gemm=True,
        qk_layernorm=bool(getattr(config, "qk_layernorm", False)),
        multi_latent_attention=bool(config.multi_latent_attention), sandwich_norm=bool(config.sandwich_norm),
        mla_qkv_concat=bool(getattr(config, "mla_qkv_concat", True)))


def get_gpt_decoder_block_spec(config) -> List[ModuleSpec]:
    """One layer spec per layer of the whole model: dense or MoE after ``config.moe_layer_pattern()``
    (``first_k_dense_replace`` wins over ``moe_layer_freq``). A pipeline stage picks its own layers from the list."""
    dense = get_gpt_layer_spec_for_config(config, False)
    moe = get_gpt_layer_spec_for_config(config, True) if config.num_moe_experts else None
    return [moe if flag else dense for flag in config.moe_layer_pattern()]


def get_gpt_mtp_block_spec(config) -> Optional[ModuleSpec]:
    """Spec of the multi-token-prediction block (None without MTP layers): every MTP layer wraps one transformer layer
    of the kind the last decoder layer has."""
    if not getattr(config, "mtp_num_layers", 0):
        return None
    pattern = config.moe_layer_pattern()
    inner = get_gpt_layer_spec_for_config(config, bool(pattern[-1]) if pattern else False)
    return ModuleSpec(module=MultiTokenPredictionBlock,
                      submodules={"layer": ModuleSpec(module=MultiTokenPredictionLayer,
                                                      submodules={"transformer_layer": inner})})
