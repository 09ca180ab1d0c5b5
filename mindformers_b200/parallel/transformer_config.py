"""Megatron-named architecture + parallelism configuration.

One dataclass carries what the reference spreads over ``ModelParallelConfig``
(``parallel_core/model_parallel_config.py:24-170``), ``MFModelConfig`` (``mf_model_config.py:74-355``)
and ``TransformerConfig`` / ``MLATransformerConfig`` (``transformer_config.py:16,400-609,613-664``).
Field names are kept so YAML files and HF-key mappings written for the reference apply unchanged;
dtype fields hold ``torch.dtype`` values after ``__post_init__``.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Union

import torch

_DTYPES = {
    "float32": torch.float32, "fp32": torch.float32, "float": torch.float32,
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float16": torch.float16, "fp16": torch.float16, "half": torch.float16,
    "float8_e4m3fn": torch.float8_e4m3fn, "fp8": torch.float8_e4m3fn,
}


def to_torch_dtype(value) -> torch.dtype:
    if isinstance(value, torch.dtype):
        return value
    if value is None:
        return torch.float32
    key = str(value).lower().replace("torch.", "").replace("mstype.", "")
    if key not in _DTYPES:
        raise ValueError(f"unknown dtype {value!r}")
    return _DTYPES[key]


@dataclass
class ModelParallelConfig:
    """Sizes of the parallel dimensions and related switches."""
    data_parallel_size: int = 1
    tensor_model_parallel_size: int = 1
    pipeline_model_parallel_size: int = 1
    virtual_pipeline_model_parallel_size: Optional[int] = None
    sequence_parallel: bool = False
    context_parallel_size: int = 1
    hierarchical_context_parallel_sizes: int = 1
    expert_model_parallel_size: int = 1
    expert_tensor_parallel_size: Optional[int] = None
    micro_batch_num: Optional[int] = 1
    seq_split_num: Optional[int] = 1
    gradient_aggregation_group: int = 4
    offset: Optional[Union[int, list]] = 0
    ulysses_degree_in_cp: int = 1
    vocab_emb_dp: Optional[bool] = True
    fp16: bool = False
    bf16: bool = False
    params_dtype: Union[str, torch.dtype] = "float32"
    finalize_model_grads_func: Optional[Callable] = None
    grad_scale_func: Optional[Callable] = None
    grad_sync_func: Optional[Callable] = None
    param_sync_func: Optional[Callable] = None
    cpu_offloading: bool = False
    cpu_offloading_num_layers: Optional[Union[list, dict]] = None
    op_swap: Optional[Union[list, dict]] = None
    default_prefetch: int = 1
    # B200 additions: which fused compute+collective paths are on
    fused_tp_comm: bool = True
    fused_moe_comm: bool = True
    fused_cp_comm: bool = True
    cp_zigzag: bool = False              # causal load balance: rank r owns sequence chunks r and 2*cp-1-r
    moe_ep_buffer_factor: float = 1.25   # row-buffer head-room over the balanced load when ep > 1

    def _check_parallel(self):
        if self.sequence_parallel and self.tensor_model_parallel_size <= 1:
            raise ValueError("sequence_parallel needs tensor_model_parallel_size > 1")
        if self.pipeline_model_parallel_size < 1 or self.tensor_model_parallel_size < 1:
            raise ValueError("parallel sizes must be >= 1")
        if self.expert_tensor_parallel_size is None:
            self.expert_tensor_parallel_size = self.tensor_model_parallel_size
        vpp = self.virtual_pipeline_model_parallel_size
        if vpp is not None and vpp > 1 and self.pipeline_model_parallel_size < 2:
            raise ValueError("virtual pipeline parallelism needs pipeline_model_parallel_size >= 2")


@dataclass
class TransformerConfig(ModelParallelConfig):
    """Architecture, numerics, MoE, recompute and long-context options of one model."""
    # ---- architecture ----
    num_layers: int = 0
    mtp_num_layers: Optional[int] = None
    mtp_loss_scaling_factor: Optional[float] = None
    hidden_size: int = 0
    num_attention_heads: int = 0
    softmax_scale: Optional[float] = None
    num_query_groups: Optional[int] = None
    ffn_hidden_size: Optional[int] = None
    kv_channels: Optional[int] = None
    hidden_dropout: float = 0.0
    attention_dropout: float = 0.0
    fp32_residual_connection: bool = False
    apply_residual_connection_post_layernorm: bool = False
    layernorm_epsilon: float = 1e-5
    layernorm_zero_centered_gamma: bool = False
    add_qkv_bias: bool = False
    add_bias_linear: bool = False
    gated_linear_unit: bool = True
    activation_func: str = "silu"
    hidden_act: str = "silu"
    normalization: str = "RMSNorm"
    qk_layernorm: bool = False
    sandwich_norm: bool = False
    num_moe_experts: Optional[int] = None
    rotary_interleaved: bool = False
    calculate_per_token_loss: bool = False
    multi_latent_attention: bool = False
    position_embedding_type: str = "rope"
    rotary_base: float = 10000.0
    rotary_percent: float = 1.0
    rotary_seq_len_interpolation_factor: Optional[float] = None
    rope_scaling: Optional[dict] = None
    use_rope_scaling: bool = False
    max_position_embeddings: int = 4096
    vocab_size: int = 128000
    seq_length: int = 4096
    pad_token_id: int = 0
    ignore_token_id: int = -100
    untie_embeddings_and_output_weights: bool = True
    tie_word_embeddings: bool = False
    post_process: bool = True
    # ---- init ----
    init_method: Optional[Callable] = None
    output_layer_init_method: Optional[Callable] = None
    init_method_std: float = 0.02
    moe_init_method_std: float = 0.01
    use_scaled_init: bool = True
    init_model_with_meta_device: bool = False
    # ---- numerics ----
    compute_dtype: Union[str, torch.dtype] = "bfloat16"
    layernorm_compute_dtype: Union[str, torch.dtype] = "float32"
    rotary_dtype: Union[str, torch.dtype] = "float32"
    softmax_compute_dtype: Union[str, torch.dtype] = "float32"
    residual_dtype: Optional[Union[str, torch.dtype]] = None
    attention_softmax_in_fp32: bool = True
    apply_query_key_layer_scaling: bool = False
    fp16_lm_cross_entropy: bool = False
    # ---- fusions (all hot ops are hand-written kernels here; the switches stay for YAML parity) ----
    bias_activation_fusion: bool = False
    bias_swiglu_fusion: bool = False
    masked_softmax_fusion: bool = False
    bias_dropout_fusion: bool = False
    apply_rope_fusion: bool = True
    persist_layer_norm: bool = False
    use_flash_attention: bool = True
    # ---- attention layout / masks ----
    input_layout: str = "BNSD"
    sparse_mode: int = 0
    use_alibi_mask: bool = False
    use_attn_mask_compression: bool = False
    use_eod_attn_mask_compression: bool = False
    use_attention_mask: bool = True
    use_eod_reset: bool = False
    use_ring_attention: bool = False
    use_contiguous_weight_layout: bool = True
    mla_qkv_concat: bool = True
    attention_pre_tokens: Optional[int] = None
    attention_next_tokens: Optional[int] = None
    context_parallel_algo: str = "colossalai_cp"
    cp_comm_type: Optional[Union[str, List[str]]] = None
    # ---- recompute ----
    recompute: Optional[Union[bool, list, tuple]] = False
    select_recompute: Optional[Union[bool, list]] = False
    parallel_optimizer_comm_recompute: Optional[Union[bool, list]] = False
    select_comm_recompute: Optional[bool] = False
    mp_comm_recompute: Optional[bool] = True
    recompute_slice_activation: bool = False
    select_recompute_exclude: Optional[Union[bool, list]] = False
    select_comm_recompute_exclude: Optional[Union[bool, list]] = False
    # ---- MoE ----
    moe_shared_expert_intermediate_size: Optional[int] = None
    moe_shared_expert_overlap: bool = False
    moe_layer_freq: Optional[Union[int, List[int]]] = 1
    first_k_dense_replace: Optional[int] = None
    moe_ffn_hidden_size: Optional[int] = None
    moe_router_load_balancing_type: str = "aux_loss"
    moe_router_topk: int = 2
    moe_router_num_groups: Optional[int] = None
    moe_router_group_topk: Optional[int] = None
    moe_router_pre_softmax: bool = False
    moe_router_topk_scaling_factor: Optional[float] = None
    moe_router_score_function: str = "softmax"
    moe_router_dtype: Union[str, torch.dtype] = "float32"
    moe_router_enable_expert_bias: bool = False
    moe_router_bias_update_rate: float = 1e-3
    moe_grouped_gemm: bool = True
    moe_aux_loss_coeff: float = 0.0
    moe_z_loss_coeff: Optional[float] = None
    moe_input_jitter_eps: Optional[float] = None
    moe_expert_capacity_factor: Optional[float] = None
    moe_pad_expert_input_to_capacity: bool = False
    moe_token_drop_policy: str = "probs"
    moe_permute_fusion: bool = True
    moe_apply_probs_on_input: bool = False
    moe_token_dispatcher_type: str = "alltoall"
    use_allgather_dispatcher: bool = False
    kv_cache_dtype: Optional[str] = None    # "int8": paged KV cache in int8 with per-token, per-head scales
    enable_deredundency: bool = False       # two-level dispatch: all-gather across nodes, all-to-all inside a node
    npu_nums_per_device: int = 1            # ranks per node for the two-level dispatch (the reference's key name)
    group_wise_a2a: bool = False
    moe_enable_deepep: bool = False
    moe_per_layer_logging: bool = False
    norm_topk_prob: bool = True
    shared_expert_num: int = 0
    use_shared_expert_gating: bool = False
    use_pad_tokens: bool = False
    aux_loss_types: Optional[list] = None
    aux_loss_factors: Optional[list] = None
    topk_method: str = "greedy"
    # ---- inference ----
    block_size: int = 16
    num_blocks: int = 512
    parallel_decoding_params: Optional[dict] = None
    is_dynamic: bool = False
    pet_config: Optional[dict] = None
    quantization: Optional[str] = None  # None | "fp8_block" (block-scaled e4m3 weights)
    # ---- MLA (filled by MLATransformerConfig) ----
    q_lora_rank: Optional[int] = None
    kv_lora_rank: int = 512
    qk_head_dim: int = 128
    qk_pos_emb_head_dim: int = 64
    v_head_dim: int = 128
    rope_type: str = "rope"
    rotary_scaling_factor: float = 1.0
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    mscale: float = 1.0
    mscale_all_dim: float = 0.0
    original_max_position_embeddings: Optional[int] = None

    def __post_init__(self):
        self._check_parallel()
        for name in ("compute_dtype", "layernorm_compute_dtype", "rotary_dtype", "softmax_compute_dtype",
                     "moe_router_dtype", "params_dtype"):
            setattr(self, name, to_torch_dtype(getattr(self, name)))
        if self.residual_dtype is not None:
            self.residual_dtype = to_torch_dtype(self.residual_dtype)
        if self.bf16:
            self.params_dtype = torch.bfloat16
        for name in ("hidden_dropout", "attention_dropout"):
            val = getattr(self, name)
            if not isinstance(val, (int, float)) or not 0 <= val < 1:
                raise ValueError(f"{name} must lie in [0, 1), got {val!r}")
        if self.pad_token_id is None:
            self.pad_token_id = 0
        self.mtp_num_layers = self.mtp_num_layers or 0
        if not isinstance(self.mtp_num_layers, int) or self.mtp_num_layers < 0:
            raise ValueError(f"mtp_num_layers must be a non-negative integer, got {self.mtp_num_layers!r}")
        if self.mtp_num_layers > 1:
            raise ValueError("only mtp_num_layers in {0, 1} is supported")
        tp = self.tensor_model_parallel_size
        if self.num_attention_heads and self.num_attention_heads % tp != 0:
            raise ValueError(f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                             f"tensor_model_parallel_size ({tp})")
        if self.ffn_hidden_size is None:
            self.ffn_hidden_size = 4 * self.hidden_size
        if self.kv_channels is None and self.num_attention_heads:
            self.kv_channels = self.hidden_size // self.num_attention_heads
        if self.num_query_groups is None:
            self.num_query_groups = self.num_attention_heads
        if self.num_query_groups and self.num_query_groups % tp != 0 and tp % self.num_query_groups != 0:
            raise ValueError(f"num_query_groups ({self.num_query_groups}) and tensor_model_parallel_size "
                             f"({tp}) must divide one another")
        if self.context_parallel_size > 1 and not self.use_flash_attention:
            raise ValueError("context parallelism needs use_flash_attention=True")
        # attention layout / sparse mode selection (reference transformer_config.py:466-487)
        if self.use_flash_attention:
            if self.use_eod_attn_mask_compression and not self.use_ring_attention:
                self.input_layout, self.sparse_mode = "TND", 3
                self.attention_dropout = 0.0
            elif self.use_attn_mask_compression and not self.use_ring_attention:
                self.sparse_mode = 2
            if self.use_ring_attention and (self.use_eod_attn_mask_compression or self.use_attn_mask_compression):
                raise ValueError("ring attention cannot be combined with attention-mask compression")
        if self.cp_comm_type is None:
            algo = self.context_parallel_algo
            self.cp_comm_type = {"colossalai_cp": "all_gather", "ulysses_cp": "a2a",
                                 "hybrid_cp": "a2a+p2p"}.get(algo, algo)
            if self.use_ring_attention:
                self.cp_comm_type = "p2p"
        # MoE
        if self.num_moe_experts:
            if self.moe_ffn_hidden_size is None:
                self.moe_ffn_hidden_size = self.ffn_hidden_size
            if self.moe_router_topk < 1 or self.moe_router_topk > self.num_moe_experts:
                raise ValueError("moe_router_topk must lie in [1, num_moe_experts]")
            if self.num_moe_experts % self.expert_model_parallel_size != 0:
                raise ValueError("num_moe_experts must be a multiple of expert_model_parallel_size")
            if self.moe_router_topk_scaling_factor is None:
                self.moe_router_topk_scaling_factor = 1.0
            if self.moe_router_score_function not in ("softmax", "sigmoid"):
                raise ValueError("moe_router_score_function must be 'softmax' or 'sigmoid'")
            if self.shared_expert_num and self.moe_shared_expert_intermediate_size is None:
                self.moe_shared_expert_intermediate_size = self.shared_expert_num * self.moe_ffn_hidden_size
            if self.first_k_dense_replace is not None and self.first_k_dense_replace > self.num_layers:
                raise ValueError("first_k_dense_replace exceeds num_layers")
            if self.aux_loss_types and self.aux_loss_factors and "expert" in self.aux_loss_types \
                    and not self.moe_aux_loss_coeff:
                self.moe_aux_loss_coeff = float(self.aux_loss_factors[self.aux_loss_types.index("expert")])
        elif self.expert_model_parallel_size > 1:
            raise ValueError("expert_model_parallel_size > 1 needs num_moe_experts")
        if self.tie_word_embeddings:
            self.untie_embeddings_and_output_weights = False
        if self.use_scaled_init and self.num_layers:
            self.output_layer_init_std = self.init_method_std / (2.0 * self.num_layers) ** 0.5
        else:
            self.output_layer_init_std = self.init_method_std
        # the initialisers themselves, for callers that pass them on (parallel/init_method.py)
        from .init_method import init_method_normal, scaled_init_method_normal
        if self.init_method is None:
            self.init_method = init_method_normal(self.init_method_std)
        if self.output_layer_init_method is None:
            self.output_layer_init_method = (scaled_init_method_normal(self.init_method_std, self.num_layers)
                                             if self.use_scaled_init and self.num_layers
                                             else init_method_normal(self.init_method_std))

    # -------------------------------------------------------------------------------------------
    @property
    def head_dim(self) -> int:
        return self.kv_channels

    def moe_layer_pattern(self) -> List[int]:
        """1 for MoE layers, 0 for dense layers (``first_k_dense_replace`` wins over ``moe_layer_freq``)."""
        if not self.num_moe_experts:
            return [0] * self.num_layers
        if self.first_k_dense_replace is not None:
            return [0 if i < self.first_k_dense_replace else 1 for i in range(self.num_layers)]
        freq = self.moe_layer_freq
        if isinstance(freq, int):
            return [1 if i % freq == 0 else 0 for i in range(self.num_layers)]
        if len(freq) != self.num_layers:
            raise ValueError("moe_layer_freq list must have num_layers entries")
        return [int(x) for x in freq]

    def to_dict(self) -> dict:
        out = {}
        for f in dataclasses.fields(self):
            v = getattr(self, f.name)
            if callable(v):
                continue
            out[f.name] = str(v).replace("torch.", "") if isinstance(v, torch.dtype) else v
        return out


@dataclass
class MLATransformerConfig(TransformerConfig):
    """Multi-latent attention (DeepSeek-V2/V3) variant with YaRN rotary parameters."""
    multi_latent_attention: bool = True
    q_lora_rank: Optional[int] = 512
    kv_lora_rank: int = 512
    qk_head_dim: int = 128
    qk_pos_emb_head_dim: int = 64
    v_head_dim: int = 128
    normalization: str = "RMSNorm"
    rope_type: str = "yarn"
    rotary_percent: float = 1.0
    rotary_scaling_factor: float = 40.0
    max_position_embeddings: int = 4096
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    mscale: float = 0.707
    mscale_all_dim: float = 0.707

    def __post_init__(self):
        super().__post_init__()
        if self.kv_lora_rank <= 0:
            raise ValueError("kv_lora_rank must be positive")
        if self.original_max_position_embeddings is None:
            self.original_max_position_embeddings = self.max_position_embeddings

    @property
    def q_head_dim(self) -> int:
        return self.qk_head_dim + self.qk_pos_emb_head_dim
