"""Plain layers of the legacy stack (``mindformers/modules/layers.py``): ``Linear`` (optionally one matrix per expert),
``LayerNorm``, ``FreqsMgr`` (rotary tables with PI / NTK / YaRN / Llama-3 context extension), ``AlibiTensor``,
``Dropout`` and the dynamic causal mask."""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as Fn
from .activation import get_activation


class Linear(nn.Module):
    """``y = act(x W^T + b)``; with ``expert_num > 1`` the weight is ``[E, out, in]`` and ``x`` is ``[E, tokens, in]``.
    ``y = act(x W^T + b)``; with ``expert_num > 1`` the weight is ``[E, out, in]`` and ``x`` is ``[E, tokens, in]``."""

    def __init__(self, in_channels: int, out_channels: int, has_bias: bool = True, activation=None, expert_num: int = 1,
                 use_gmm: bool = False, transpose_b: bool = True, param_init_type=torch.float32, compute_dtype=torch.bfloat16,
                 weight_init_std: float = 0.02, device=None):
        super().__init__()
        self.expert_num, self.compute_dtype = expert_num, compute_dtype
        shape = (out_channels, in_channels) if expert_num == 1 else (expert_num, out_channels, in_channels)
        self.weight = nn.Parameter(torch.empty(shape, dtype=param_init_type, device=device).normal_(0, weight_init_std))
        bshape = (out_channels,) if expert_num == 1 else (expert_num, 1, out_channels)
        self.bias = nn.Parameter(torch.zeros(bshape, dtype=param_init_type, device=device)) if has_bias else None
        self.activation = get_activation(activation) if isinstance(activation, str) else activation

    def forward(self, x):
        dt = x.dtype
        w = self.weight.to(self.compute_dtype)
        xc = x.to(self.compute_dtype)
        if self.expert_num == 1:
            y = Fn.linear(xc.reshape(-1, xc.shape[-1]), w).reshape(*x.shape[:-1], w.shape[0]) if xc.is_cuda and w.dtype == torch.bfloat16 \
                else F.linear(xc, w)
        else:
            y = torch.bmm(xc, w.transpose(1, 2))
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        if self.activation is not None:
            y = self.activation(y)
        return y.to(dt)


class LayerNorm(nn.Module):
    """LayerNorm with the legacy stack's argument names (``normalized_shape``, ``eps``, ``param_init_type``); fp32
    statistics."""

    def __init__(self, normalized_shape, eps: float = 1e-5, param_init_type=torch.float32, device=None):
        super().__init__()
        shape = (normalized_shape,) if isinstance(normalized_shape, int) else tuple(normalized_shape)
        self.gamma = nn.Parameter(torch.ones(shape, dtype=param_init_type, device=device))
        self.beta = nn.Parameter(torch.zeros(shape, dtype=param_init_type, device=device))
        self.eps = eps

    def forward(self, x):
        return F.layer_norm(x.float(), self.gamma.shape, self.gamma.float(), self.beta.float(), self.eps).to(x.dtype)


class Dropout(nn.Module):
    """Dropout configured by keep probability, as the legacy layers do (``keep_prob=1`` is the identity)."""

    def __init__(self, keep_prob: float = 1.0):
        super().__init__()
        self.p = 1.0 - keep_prob

    def forward(self, x):
        return F.dropout(x, self.p, self.training) if self.p > 0 else x


class LowerTriangularMaskWithDynamic(nn.Module):
    """Causal mask for a batch of (padded) sequences: 1 = masked, as the legacy attention expects."""

    def __init__(self, seq_length: int, pad_token_id: int = 0, compute_type=torch.float16):
        super().__init__()
        self.pad, self.dtype = pad_token_id, compute_type
        self.register_buffer("tril", torch.tril(torch.ones(seq_length, seq_length)), persistent=False)

    def forward(self, tokens: torch.Tensor, masks: Optional[torch.Tensor] = None):
        B, S = tokens.shape
        valid = (tokens != self.pad).to(self.tril.dtype) if masks is None else masks.to(self.tril.dtype)
        m = valid[:, None, :] * valid[:, :, None] * self.tril[:S, :S].to(tokens.device)
        return (1.0 - m).to(self.dtype)


class FreqsMgr(nn.Module):
    """Rotary ``cos`` / ``sin`` tables ``[max_pos, head_dim]`` with the context-extension methods of the legacy stack:
    ``NONE``, ``PI`` (position interpolation), ``NTK`` (base rescaling), ``YARN``, ``LLAMA3`` (frequency-band scaling)."""

    def __init__(self, head_dim: int, seq_length: int, max_position_embedding: int = 4096, theta: float = 10000.0,
                 scaling_factor: float = 1.0, extend_method: str = "NONE", rotary_dtype=torch.float32, parallel_config=None,
                 low_freq_factor: float = 1.0, high_freq_factor: float = 4.0, original_max_position: int = 8192,
                 beta_fast: float = 32.0, beta_slow: float = 1.0, mscale: float = 1.0, device=None):
        super().__init__()
        method = str(extend_method).upper()
        half = torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim
        base = theta
        if method == "NTK":
            base = theta * scaling_factor ** (head_dim / (head_dim - 2))
        inv = 1.0 / (base ** half)
        self.mscale = 1.0
        if method == "LLAMA3":
            wavelen = 2 * math.pi / inv
            low, high = original_max_position / low_freq_factor, original_max_position / high_freq_factor
            smooth = ((original_max_position / wavelen) - low_freq_factor) / (high_freq_factor - low_freq_factor)
            mid = (1 - smooth) * inv / scaling_factor + smooth * inv
            inv = torch.where(wavelen > low, inv / scaling_factor, torch.where(wavelen < high, inv, mid))
        elif method == "YARN":
            def corr(n_rot):
                return head_dim * math.log(original_max_position / (n_rot * 2 * math.pi)) / (2 * math.log(theta))
            lo, hi = max(math.floor(corr(beta_fast)), 0), min(math.ceil(corr(beta_slow)), head_dim // 2 - 1)
            ramp = ((torch.arange(head_dim // 2, dtype=torch.float32, device=device) - lo) / max(hi - lo, 1e-3)).clamp(0, 1)
            inv = inv / scaling_factor * ramp + inv * (1 - ramp)
            self.mscale = (0.1 * mscale * math.log(scaling_factor) + 1.0) if scaling_factor > 1 else 1.0
        t = torch.arange(0, max(seq_length, max_position_embedding), dtype=torch.float32, device=device)
        if method == "PI":
            t = t / scaling_factor
        freqs = torch.outer(t, inv)
        emb = torch.cat((freqs, freqs), dim=-1)
        self.register_buffer("freqs_cos", (emb.cos() * self.mscale).to(rotary_dtype), persistent=False)
        self.register_buffer("freqs_sin", (emb.sin() * self.mscale).to(rotary_dtype), persistent=False)
        self.head_dim = head_dim

    def forward(self, seq_length: Optional[int] = None):
        n = seq_length or self.freqs_cos.shape[0]
        return self.freqs_cos[:n], self.freqs_sin[:n]

    def increment(self, batch_valid_length: torch.Tensor):
        idx = (batch_valid_length - 1).long()
        return self.freqs_cos.index_select(0, idx), self.freqs_sin.index_select(0, idx)

    def prefill(self, bs: int, seq_length: int):
        return self.freqs_cos[:seq_length].repeat(bs, 1), self.freqs_sin[:seq_length].repeat(bs, 1)


def rotate_half(x):
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def apply_rotary(x, cos, sin):
    """``x [..., S, D]`` with tables ``[S, D]`` (rotate-half convention)."""
    return x * cos + rotate_half(x) * sin


class AlibiTensor(nn.Module):
    """Attention bias ``slope_h * (key_pos - query_pos)`` per head (``AlibiTensorV2`` semantics: computed from
    positions)."""

    def __init__(self, seq_length: int, num_heads: int):
        super().__init__()
        n = 2 ** math.floor(math.log2(num_heads))
        base = 2.0 ** (-(2.0 ** -(math.log2(n) - 3)))
        slopes = torch.pow(base, torch.arange(1, n + 1, dtype=torch.float32))
        if n != num_heads:
            extra = 2.0 ** (-(2.0 ** -(math.log2(2 * n) - 3)))
            slopes = torch.cat([slopes, torch.pow(extra, torch.arange(1, 2 * (num_heads - n) + 1, 2, dtype=torch.float32))])
        self.register_buffer("slopes", slopes.view(1, num_heads, 1, 1), persistent=False)

    def forward(self, attention_mask: torch.Tensor, dtype=torch.float32):
        """``attention_mask [B, S]`` (1 = token) → bias ``[B, H, 1, S]``."""
        pos = ((attention_mask.cumsum(-1) - 1) * attention_mask).to(torch.float32)
        return (self.slopes.to(pos.device) * pos[:, None, None, :]).to(dtype)


class AlibiTensorV2(nn.Module):
    """ALiBi bias from a token mask (reference ``modules/layers.py`` ``AlibiTensorV2``): ``attention_mask [B, S]`` (1 = token)
    gives ``[B, num_heads, 1, S]`` with ``slope_h * (number of earlier tokens)`` at every token and 0 at padding, so
    left- or right-padded batches get the distances of their real tokens."""

    def __init__(self, num_heads: int):
        super().__init__()
        self.num_heads = num_heads
        closest = 2 ** math.floor(math.log2(num_heads))
        base = 2.0 ** (-(2.0 ** -(math.log2(closest) - 3)))
        slopes = [base ** (i + 1) for i in range(closest)]
        if closest != num_heads:
            extra = 2.0 ** (-(2.0 ** -(math.log2(2 * closest) - 3)))
            slopes += [extra ** (i + 1) for i in range(0, 2 * (num_heads - closest), 2)]
        self.register_buffer("slopes", torch.tensor(slopes, dtype=torch.float32), persistent=False)

    def forward(self, attention_mask: torch.Tensor, dtype=torch.float32):
        m = attention_mask.to(torch.float32)
        position = (m.cumsum(-1) - 1.0) * m                                   # [B, S]
        return (self.slopes.to(m.device)[None, :, None, None] * position[:, None, None, :]).to(dtype)


class AttentionMaskHF(nn.Module):
    """Causal mask in the convention of the older attention cells (reference ``modules/transformer/transformer.py``
    ``AttentionMaskHF``): ``input_mask [B, S]`` (1 = token) gives ``[B, S, S]`` with 1 where query i may attend key j
    (j <= i and both are tokens)."""

    def __init__(self, seq_length: int, compute_dtype=torch.float32):
        super().__init__()
        self.seq_length, self.dtype = seq_length, compute_dtype
        self.register_buffer("tril", torch.tril(torch.ones(seq_length, seq_length)), persistent=False)

    def forward(self, input_mask: torch.Tensor):
        m = input_mask.to(self.dtype)
        s = m.shape[-1]
        return m[:, :, None] * m[:, None, :] * self.tril[:s, :s].to(m.device, self.dtype)


class RotaryEmbedding(nn.Module):
    """Applies rotary position embedding to query and key (reference ``modules/layers.py:1461``): ``xq, xk`` are
    ``[B, heads, S, head_dim]``, ``freqs_cis = (cos, sin, swap_mask)`` as ``FreqsMgr`` returns them (``cos`` / ``sin``
    ``[S, head_dim]``; the third entry is unused, the half rotation is done by slicing)."""

    def __init__(self, head_dim: int = 128, compute_dtype=torch.float32, use_rope_slice: bool = False, **kwargs):
        super().__init__()
        self.head_dim, self.dtype = head_dim, compute_dtype

    @staticmethod
    def rotate_half(x):
        a, b = x.chunk(2, dim=-1)
        return torch.cat((-b, a), dim=-1)

    def forward(self, xq: torch.Tensor, xk: torch.Tensor, freqs_cis):
        cos, sin = freqs_cis[0], freqs_cis[1]
        out = []
        for x in (xq, xk):
            xf = x.to(self.dtype)
            out.append((xf * cos.to(self.dtype) + self.rotate_half(xf) * sin.to(self.dtype)).to(x.dtype))
        return out[0], out[1]
