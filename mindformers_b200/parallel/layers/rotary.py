"""Rotary position embedding tables: plain, Llama-3 frequency scaling and YaRN.

Reference: ``training_graph/base_models/common/embeddings/rotary_pos_embedding.py`` (:29-147, Llama-3
scaling ``_apply_scaling`` :79-104), ``yarn_rotary_pos_embedding.py`` (:32, helpers :138-166) and the
inference caches in ``inference/base_models/common/embeddings/rotary_pos_embedding.py`` (:33-211).
The tables are ``cos/sin [max_positions, rot/2]`` in fp32; the kernel in ``ops`` applies them in
place to q and k (rotate-half or interleaved pairs).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn


def _llama3_scale(inv_freq: torch.Tensor, factor=8.0, low=1.0, high=4.0, original=8192) -> torch.Tensor:
    wavelen = 2 * math.pi / inv_freq
    low_wl, high_wl = original / low, original / high
    smooth = (original / wavelen - low) / (high - low)
    mid = (1 - smooth) * inv_freq / factor + smooth * inv_freq
    out = torch.where(wavelen > low_wl, inv_freq / factor, inv_freq)
    is_mid = (wavelen <= low_wl) & (wavelen >= high_wl)
    return torch.where(is_mid, mid, out)


def yarn_find_correction_dim(num_rotations, dim, base, max_pos):
    return (dim * math.log(max_pos / (num_rotations * 2 * math.pi))) / (2 * math.log(base))


def yarn_find_correction_range(low_rot, high_rot, dim, base, max_pos):
    low = math.floor(yarn_find_correction_dim(low_rot, dim, base, max_pos))
    high = math.ceil(yarn_find_correction_dim(high_rot, dim, base, max_pos))
    return max(low, 0), min(high, dim - 1)


def yarn_linear_ramp_mask(lo, hi, dim):
    if lo == hi:
        hi += 0.001
    ramp = (torch.arange(dim, dtype=torch.float32) - lo) / (hi - lo)
    return ramp.clamp(0, 1)


def yarn_get_mscale(scale: float = 1.0, mscale: float = 1.0) -> float:
    if scale <= 1:
        return 1.0
    return 0.1 * mscale * math.log(scale) + 1.0


class RotaryEmbedding(nn.Module):
    """Precomputed cos/sin tables.

    Args: ``kv_channels`` (head dim), ``rotary_percent``, ``rotary_base``, ``rope_scaling`` (HF-style dict,
    ``{"rope_type": "llama3", "factor": 8, ...}``), ``seq_len_interpolation_factor`` (position interpolation).
    """

    def __init__(self, kv_channels: int, rotary_percent: float = 1.0, rotary_base: float = 10000.0,
                 max_positions: int = 4096, rope_scaling: Optional[dict] = None,
                 seq_len_interpolation_factor: Optional[float] = None, device=None):
        super().__init__()
        dim = int(kv_channels * rotary_percent)
        dim -= dim % 2
        self.rot_dim = dim
        inv = 1.0 / (rotary_base ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
        self.mscale = 1.0
        if rope_scaling:
            kind = rope_scaling.get("rope_type", rope_scaling.get("type"))
            if kind == "llama3":
                inv = _llama3_scale(inv, rope_scaling.get("factor", 8.0), rope_scaling.get("low_freq_factor", 1.0),
                                    rope_scaling.get("high_freq_factor", 4.0),
                                    rope_scaling.get("original_max_position_embeddings", 8192))
            elif kind == "linear":
                inv = inv / rope_scaling.get("factor", 1.0)
        pos = torch.arange(max_positions, dtype=torch.float32)
        if seq_len_interpolation_factor:
            pos = pos / seq_len_interpolation_factor
        ang = pos[:, None] * inv[None, :]
        self.register_buffer("cos", ang.cos().contiguous().to(device), persistent=False)
        self.register_buffer("sin", ang.sin().contiguous().to(device), persistent=False)

    def forward(self) -> Tuple[torch.Tensor, torch.Tensor]:
        return self.cos, self.sin


class YarnRotaryEmbedding(RotaryEmbedding):
    """YaRN: frequency-dependent interpolation plus the attention ``mscale`` (DeepSeek-V2/V3)."""

    def __init__(self, kv_channels: int, rotary_base: float = 10000.0, scaling_factor: float = 1.0,
                 original_max_position_embeddings: int = 4096, beta_fast: float = 32.0, beta_slow: float = 1.0,
                 mscale: float = 1.0, mscale_all_dim: float = 0.0, max_positions: int = 4096, device=None):
        nn.Module.__init__(self)
        dim = kv_channels - kv_channels % 2
        self.rot_dim = dim
        exps = torch.arange(0, dim, 2, dtype=torch.float32) / dim
        inv_extra = 1.0 / (rotary_base ** exps)
        inv_inter = 1.0 / (scaling_factor * rotary_base ** exps)
        lo, hi = yarn_find_correction_range(beta_fast, beta_slow, dim, rotary_base, original_max_position_embeddings)
        mask = 1.0 - yarn_linear_ramp_mask(lo, hi, dim // 2)
        inv = inv_inter * (1 - mask) + inv_extra * mask
        self.mscale = yarn_get_mscale(scaling_factor, mscale) / yarn_get_mscale(scaling_factor, mscale_all_dim)
        pos = torch.arange(max_positions, dtype=torch.float32)
        ang = pos[:, None] * inv[None, :]
        self.register_buffer("cos", (ang.cos() * self.mscale).contiguous().to(device), persistent=False)
        self.register_buffer("sin", (ang.sin() * self.mscale).contiguous().to(device), persistent=False)


def get_rope(config, max_positions: Optional[int] = None, head_dim: Optional[int] = None, device=None):
    """Build the rotary table a model configuration asks for."""
    maxp = max_positions or max(config.max_position_embeddings, config.seq_length)
    if config.multi_latent_attention:
        hd = config.qk_pos_emb_head_dim
        if config.rope_type == "yarn" and config.rotary_scaling_factor and config.rotary_scaling_factor > 1:
            return YarnRotaryEmbedding(hd, config.rotary_base, config.rotary_scaling_factor,
                                       config.original_max_position_embeddings or config.max_position_embeddings,
                                       config.beta_fast, config.beta_slow, config.mscale, config.mscale_all_dim,
                                       max_positions=maxp, device=device)
        return RotaryEmbedding(hd, 1.0, config.rotary_base, maxp, None, None, device=device)
    hd = head_dim or config.kv_channels
    scaling = config.rope_scaling if (config.use_rope_scaling or config.rope_scaling) else None
    return RotaryEmbedding(hd, config.rotary_percent, config.rotary_base, maxp, scaling,
                           config.rotary_seq_len_interpolation_factor, device=device)
