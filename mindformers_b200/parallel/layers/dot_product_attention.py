"""Unfused attention path: mask generation, scale-mask-softmax and the dot-product core attention.

Reference: ``training_graph/transformer/mask_generate.py:26`` (``CausalMaskGenerate``: a full ``[S, S]`` mask or the
2048 x 2048 compressed one that the flash-attention op expands), ``fused_softmax.py:27`` (``FusedScaleMaskSoftmax``:
scale, mask fill, softmax in fp32, cast back), ``utils.py:28`` (``AttnMaskFill``) and the inference
``dot_product_attention.py`` / ``lower_triangular_mask.py`` (128 x 128 prefill mask, 1 x 1 decode mask).

The flash-attention kernel (``ops/csrc/flash_attention.cu``) serves every configuration with ``use_flash_attention``
(the default). This module is the path for ``use_flash_attention=False`` and for arbitrary masks, which the kernel does
not take: an explicit additive mask, padding masks, or the per-document mask after an end-of-document reset. Mask
convention as in the reference: 1 (True) = masked.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn

COMPRESSED_MASK_SIZE = 2048


class CausalMaskGenerate(nn.Module):
    """Causal mask of a ``[B, S]`` batch. ``compressed=True`` returns the fixed 2048 x 2048 upper-triangular mask that
    stands for "causal at any length". With ``position_ids`` that restart inside a row (end-of-document reset) or with
    ``actual_seq_len`` (cumulative segment ends) tokens only see their own document."""

    def __init__(self, seq_length: int, compressed: bool = False, pad_token_id: Optional[int] = None,
                 dtype=torch.bool):
        super().__init__()
        self.seq_length, self.compressed, self.pad, self.dtype = seq_length, compressed, pad_token_id, dtype
        n = COMPRESSED_MASK_SIZE if compressed else seq_length
        self.register_buffer("triu", torch.ones(n, n, dtype=torch.bool).triu(1), persistent=False)

    def forward(self, tokens: Optional[torch.Tensor] = None, position_ids: Optional[torch.Tensor] = None,
                actual_seq_len: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.compressed:
            return self.triu.to(self.dtype)
        if tokens is None and position_ids is None and actual_seq_len is None:
            return self.triu.to(self.dtype)
        ref = tokens if tokens is not None else position_ids
        B, S = ref.shape[0], ref.shape[1]
        mask = self.triu[:S, :S].to(ref.device).unsqueeze(0).expand(B, S, S).clone()
        if position_ids is not None:            # a document starts where the position goes back to 0
            starts = (position_ids == 0).long()
            doc = starts.cumsum(-1)
            mask |= doc.unsqueeze(-1) != doc.unsqueeze(-2)
        if actual_seq_len is not None:          # cumulative ends of the packed segments of every row
            ends = actual_seq_len.to(ref.device).reshape(B, -1)
            idx = torch.arange(S, device=ref.device)
            doc = (idx.view(1, S, 1) >= ends.unsqueeze(1)).sum(-1)
            mask |= doc.unsqueeze(-1) != doc.unsqueeze(-2)
        if tokens is not None and self.pad is not None:
            pad = tokens == self.pad
            mask |= pad.unsqueeze(-1) | pad.unsqueeze(-2)
        return mask.unsqueeze(1).to(self.dtype)                    # [B, 1, S, S]


class AttnMaskFill(nn.Module):
    """``scores`` with the masked positions set to ``value`` (mask: 1 / True = masked, broadcastable)."""

    def __init__(self, value: float = -10000.0):
        super().__init__()
        self.value = value

    def forward(self, scores: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        return scores.masked_fill(mask.to(torch.bool), self.value)


class FusedScaleMaskSoftmax(nn.Module):
    """``softmax(scale * scores masked)`` computed in fp32 (``softmax_compute_dtype``) and cast back."""

    def __init__(self, scale: Optional[float] = None, softmax_in_fp32: bool = True, mask_value: float = -10000.0):
        super().__init__()
        self.scale, self.fp32 = scale, softmax_in_fp32
        self.fill = AttnMaskFill(mask_value)

    def forward(self, scores: torch.Tensor, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        dtype = scores.dtype
        x = scores.float() if self.fp32 else scores
        if self.scale is not None:
            x = x * self.scale
        if mask is not None:
            x = self.fill(x, mask)
        return torch.softmax(x, dim=-1).to(dtype)


class DotProductAttention(nn.Module):
    """``[B, S, heads, d]`` query / key / value → ``[B, S, heads * dv]`` with an explicit mask; grouped-query heads are
    repeated, attention dropout is applied to the probabilities."""

    def __init__(self, config, layer_number: int = 1, softmax_scale: Optional[float] = None, head_dim=None):
        super().__init__()
        hd = head_dim or config.kv_channels
        scale = softmax_scale if softmax_scale is not None else (config.softmax_scale or 1.0 / math.sqrt(hd))
        self.softmax = FusedScaleMaskSoftmax(scale, softmax_in_fp32=True)
        self.dropout = nn.Dropout(float(getattr(config, "attention_dropout", 0.0) or 0.0))
        self.mask = CausalMaskGenerate(config.seq_length or config.max_position_embeddings or 2048)

    def forward(self, q, k, v, attention_mask: Optional[torch.Tensor] = None, position_ids=None, actual_seq_len=None):
        B, S, nq, _ = q.shape
        rep = nq // k.shape[2]
        qh = q.permute(0, 2, 1, 3)
        kh = k.permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
        vh = v.permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
        if attention_mask is None:
            if position_ids is None and actual_seq_len is None:
                attention_mask = torch.ones(S, S, dtype=torch.bool, device=q.device).triu(1)
            else:
                if position_ids is None:
                    position_ids = torch.arange(S, device=q.device).unsqueeze(0).expand(B, S)
                attention_mask = self.mask(position_ids=position_ids, actual_seq_len=actual_seq_len)
        probs = self.dropout(self.softmax(torch.matmul(qh, kh.transpose(-1, -2)), attention_mask))
        out = torch.matmul(probs.to(vh.dtype), vh)
        return out.permute(0, 2, 1, 3).reshape(B, S, -1)


class LowerTriangularMask(nn.Module):
    """Inference masks: a fixed 128 x 128 causal mask for prefill (the attention op tiles it) and a 1 x 1 zero mask for
    decode."""

    def __init__(self, dtype=torch.bfloat16, size: int = 128):
        super().__init__()
        self.register_buffer("prefill_mask", torch.ones(size, size).triu(1).to(dtype), persistent=False)
        self.register_buffer("decode_mask", torch.zeros(1, 1, dtype=dtype), persistent=False)

    def forward(self, is_prefill: bool) -> torch.Tensor:
        return self.prefill_mask if is_prefill else self.decode_mask
