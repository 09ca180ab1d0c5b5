"""Small building blocks and spec containers that the reference's ``parallel_core`` layer files define beside the layers.

* ``IdentityOp`` / ``IdentityFuncOp`` (``transformer/identity_op.py``): stand-ins for a spec entry that is left out.
* ``AttnMaskType`` (``transformer/enums.py``).
* ``*Submodules`` dataclasses (``transformer/attention.py``, ``multi_latent_attention.py``, ``mlp.py``,
  ``moe/moe_layer.py``, ``transformer_block.py``, ``multi_token_prediction.py``): what a module is composed of, as
  ``ModuleSpec`` entries.
* ``get_act_func`` (``transformer/activation.py``), ``get_norm_cls`` (``transformer/norm.py``), ``get_attn_mask_func``
  (``transformer/utils.py``).
* ``SwiGlu`` (``training_graph/activation.py``) and ``ApplyRotaryPosEmb`` (``embeddings/rope_utils.py``) as modules over
  the fused kernels of ``ops/functional.py``.
* ``Router`` (``moe/router.py``) and ``MoETokenDispatcher`` (``moe/token_dispatcher.py``): the abstract bases of
  ``TopKRouter`` and the dispatchers.
* the tensor-parallel mapping cells of the inference tree (``inference/tensor_parallel/mappings.py``).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Any, List, Optional

import torch
import torch.nn as nn

from ...ops import functional as Fn
from .. import mappings as M
from .. import parallel_state as ps
from . import norm as _norm


class IdentityOp(nn.Module):
    """Returns its first argument unchanged (a spec entry that is switched off, e.g. no q/k layer norm)."""

    def __init__(self, *args, **kwargs):
        super().__init__()

    def forward(self, x, *args, **kwargs):
        return x


class IdentityFuncOp(IdentityOp):
    """Returns a function that returns its argument (the form ``bias_dropout_add`` style entries expect)."""

    def forward(self, *args, **kwargs):
        return super().forward


class AttnMaskType(enum.Enum):
    padding = 1
    causal = 2
    no_mask = 3
    padding_causal = 4
    arbitrary = 5


@dataclass
class SelfAttentionSubmodules:
    linear_qkv: Any = None
    core_attention: Any = None
    linear_proj: Any = None
    q_layernorm: Any = None
    k_layernorm: Any = None


@dataclass
class CrossAttentionSubmodules:
    linear_q: Any = None
    linear_kv: Any = None
    core_attention: Any = None
    linear_proj: Any = None


@dataclass
class MLASelfAttentionSubmodules:
    linear_q_proj: Any = None
    linear_q_down_proj: Any = None
    linear_q_up_proj: Any = None
    linear_kv_down_proj: Any = None
    linear_kv_up_proj: Any = None
    core_attention: Any = None
    linear_proj: Any = None
    q_layernorm: Any = None
    kv_layernorm: Any = None


@dataclass
class MLASelfAttentionSubmodulesConcatenated:
    """Variant whose q and kv down-projections are one matrix (``linear_qkv``)."""
    linear_qkv: Any = None
    linear_qb: Any = None
    linear_kvb: Any = None
    core_attention: Any = None
    linear_proj: Any = None
    q_layernorm: Any = None
    k_layernorm: Any = None


@dataclass
class MLPSubmodules:
    linear_fc1: Any = None
    linear_fc2: Any = None


@dataclass
class MoESubmodules:
    experts: Any = None
    shared_experts: Any = None


@dataclass
class TransformerBlockSubmodules:
    layer_specs: List[Any] = field(default_factory=list)
    layer_norm: Any = None


@dataclass
class MultiTokenPredictionLayerSubmodules:
    enorm: Any = None
    hnorm: Any = None
    eh_proj: Any = None
    transformer_layer: Any = None
    layer_norm: Any = None


@dataclass
class MultiTokenPredictionBlockSubmodules:
    layer_specs: List[Any] = field(default_factory=list)


class SwiGlu(nn.Module):
    """``silu(x[..., :h]) * x[..., h:]`` on the packed gate/up projection (the fused kernel on a GPU)."""

    def forward(self, x):
        return Fn.swiglu(x)


_ACTIVATIONS = {
    "gelu": lambda: nn.GELU(), "fast_gelu": lambda: nn.GELU(approximate="tanh"), "silu": lambda: nn.SiLU(), "swish": lambda: nn.SiLU(),
    "swiglu": lambda: SwiGlu(), "relu": lambda: nn.ReLU(), "sigmoid": lambda: nn.Sigmoid(), "squared_relu": None,
}


class _SquaredReLU(nn.Module):
    def forward(self, x):
        return torch.relu(x) ** 2


def get_act_func(activation_type: str, *args, **kwargs) -> nn.Module:
    """Activation module by name (case-insensitive): gelu, fast_gelu, silu / swish, swiglu, relu, sigmoid, squared_relu."""
    key = str(activation_type).lower()
    if key == "squared_relu":
        return _SquaredReLU()
    if key not in _ACTIVATIONS:
        raise NotImplementedError(f"activation {activation_type!r} is not one of {sorted(_ACTIVATIONS)}")
    return _ACTIVATIONS[key]()


def get_norm_cls(normalization: str, fused_kernel: bool = True):
    """Norm class by name (``LayerNorm`` / ``RMSNorm`` and their ``Fused`` spellings: both map to the fused kernels)."""
    if normalization in ("RMSNorm", "FusedRMSNorm"):
        return _norm.RMSNorm
    if normalization in ("LayerNorm", "FusedLayerNorm"):
        return _norm.LayerNorm
    raise ValueError(f"unknown normalization {normalization!r}")


def _mask_fill(scores: torch.Tensor, mask: torch.Tensor, value: float):
    return scores.masked_fill(mask.to(torch.bool), value)


def get_attn_mask_func(mask_func_type: str):
    """``attn_mask_fill`` sets masked scores (mask = 1) to -10000; ``attn_mask_add`` adds ``mask * -10000``."""
    if mask_func_type == "attn_mask_fill":
        return lambda scores, mask: _mask_fill(scores, mask, -10000.0)
    if mask_func_type == "attn_mask_add":
        return lambda scores, mask: scores + mask.to(scores.dtype) * -10000.0
    raise KeyError(f"mask function {mask_func_type!r} is not one of attn_mask_fill / attn_mask_add")


class ApplyRotaryPosEmb(nn.Module):
    """Rotary embedding of ``t [S, B, heads, hd]`` (or ``[T, heads, hd]``) with angles ``freqs [S, 1, 1, rot]``: the first
    ``rot`` dims are rotated by halves (``rotary_interleaved``: by adjacent pairs), the rest pass through; ``mscale``
    multiplies cos and sin (YaRN)."""

    def __init__(self, config=None, for_k_pos_emb: bool = False):
        super().__init__()
        self.interleaved = bool(getattr(config, "rotary_interleaved", False)) if config is not None else False

    def forward(self, t: torch.Tensor, freqs, rotary_interleaved: Optional[bool] = None, multi_latent_attention: bool = False):
        mscale = 1.0
        if isinstance(freqs, (tuple, list)):
            freqs, mscale = freqs[0], float(freqs[1])
        inter = self.interleaved if rotary_interleaved is None else rotary_interleaved
        ang = freqs.reshape(freqs.shape[0], -1).float()                 # [S, rot]: every angle appears twice
        rot = ang.shape[-1]
        base = ang[:, 0::2] if inter else ang[:, : rot // 2]            # [S, rot / 2]
        cos, sin = torch.cos(base) * mscale, torch.sin(base) * mscale
        shape = t.shape
        S = shape[0]
        flat = t.reshape(S, -1, shape[-2], shape[-1])                   # [S, B, heads, hd]
        B = flat.shape[1]
        positions = torch.arange(S, device=t.device).repeat_interleave(B)
        out = Fn.rope(flat.reshape(S * B, shape[-2], shape[-1]).contiguous(), cos, sin, positions, shape[-2], rot, inter)
        return out.reshape(shape)


class Router(nn.Module):
    """Base of the routers: owns the gate weight ``[num_experts, hidden]``; ``routing(logits)`` is the subclass's rule."""

    def __init__(self, config):
        super().__init__()
        self.config = config
        self.num_experts = config.num_moe_experts
        self.topk = config.moe_router_topk

    def gating(self, x: torch.Tensor) -> torch.Tensor:
        return torch.nn.functional.linear(x.float(), self.weight.float())

    def routing(self, logits: torch.Tensor):
        raise NotImplementedError

    def forward(self, x: torch.Tensor):
        return self.routing(self.gating(x))


class MoETokenDispatcher:
    """Interface of the token dispatchers: ``token_permutation`` moves tokens to their experts' ranks in expert order,
    ``token_unpermutation`` brings the expert outputs back and combines them with the routing weights."""

    def __init__(self, config):
        self.config = config

    def token_permutation(self, tokens, probs, routing_map):
        raise NotImplementedError

    def token_unpermutation(self, expert_output, *args, **kwargs):
        raise NotImplementedError


# ---- tensor-parallel mapping cells (inference tree) -------------------------------------------------------------------
class GatherFromModelParallelRegion(nn.Module):
    """All-gather along the last dim over the tensor-parallel group."""

    def forward(self, x):
        return M.gather_from_tensor_model_parallel_region(x) if ps.get_tensor_model_parallel_world_size() > 1 else x


class ReduceFromModelParallelRegion(nn.Module):
    def forward(self, x):
        return M.reduce_from_tensor_model_parallel_region(x) if ps.get_tensor_model_parallel_world_size() > 1 else x


class ReduceScatterToModelParallelRegion(nn.Module):
    """Sum over the group, each rank keeps its slice of the first dim."""

    def forward(self, x):
        return M.reduce_scatter_to_sequence_parallel_region(x) if ps.get_tensor_model_parallel_world_size() > 1 else x


class ScatterToModelParallelRegion(nn.Module):
    """Keeps this rank's slice of the last dim."""

    def forward(self, x):
        world = ps.get_tensor_model_parallel_world_size()
        if world == 1:
            return x
        rank = ps.get_tensor_model_parallel_rank()
        return x.chunk(world, dim=-1)[rank].contiguous()


def gather_from_model_parallel_region(x):
    return GatherFromModelParallelRegion()(x)


def reduce_from_model_parallel_region(x):
    return ReduceFromModelParallelRegion()(x)


def reduce_scatter_to_model_parallel_region(x):
    return ReduceScatterToModelParallelRegion()(x)


def scatter_to_model_parallel_region(x):
    return ScatterToModelParallelRegion()(x)
