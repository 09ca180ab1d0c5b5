"""Causal sliding-window attention computed block by block.

Reference: ``mindformers/modules/local_block_sparse_attention.py:146`` (``LocalBlockSparseAttention(seq_len,
size_per_head, local_size, block_size)``: the "local" pattern of Longformer on block granularity — the upper triangle
and the far lower triangle are never computed).

A query block of ``block_size`` tokens attends to the ``local_size / block_size`` key blocks that end with its own
(causal inside the diagonal block, and further limited by ``attention_mask`` when one is given). The key blocks of every
query block are gathered into a window tensor, so work and memory are ``O(S * local_size)`` instead of ``O(S^2)``.
Tensors are ``[batch, heads, seq, head_dim]`` as in the reference; the mask convention follows the legacy stack here:
``attention_mask [batch, seq, seq]`` with 1 = may attend.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F


class LocalBlockSparseAttention(nn.Module):
    """``forward(q, k, v, attention_mask=None)`` on ``[batch, heads, seq, head_dim]``: every query block attends to
    the ``local_size / block_size`` key blocks ending with its own, causally inside the diagonal block."""

    def __init__(self, seq_len: int, size_per_head: int, local_size: int, block_size: int, dropout_rate: float = 0.1,
                 softmax_compute_type=torch.float32, parallel_config=None):
        super().__init__()
        if seq_len % block_size or local_size % block_size:
            raise ValueError("seq_len and local_size must be multiples of block_size")
        if local_size > seq_len:
            raise ValueError("local_size must not exceed seq_len")
        self.seq_len, self.hd, self.block = seq_len, size_per_head, block_size
        self.window_blocks = local_size // block_size
        self.scale = 1.0 / math.sqrt(size_per_head)
        self.softmax_dtype = softmax_compute_type
        self.dropout = nn.Dropout(dropout_rate)
        nb, w = seq_len // block_size, self.window_blocks
        # key block index of every (query block, window slot); slots before the sequence start point at block 0 and
        # are masked out
        idx = torch.arange(nb).unsqueeze(1) - (w - 1) + torch.arange(w).unsqueeze(0)          # [nb, w]
        self.register_buffer("kv_index", idx.clamp_min(0), persistent=False)
        self.register_buffer("slot_valid", idx >= 0, persistent=False)
        causal = torch.ones(block_size, block_size, dtype=torch.bool).tril()
        allow = torch.ones(w, block_size, block_size, dtype=torch.bool)
        allow[-1] = causal                                 # the diagonal block is causal, earlier ones are fully visible
        self.register_buffer("in_window", allow, persistent=False)

    def allowed(self) -> torch.Tensor:
        """``[nb, block, w, block]`` bool: which (query, window key) pairs the pattern keeps."""
        a = self.in_window.permute(1, 0, 2).unsqueeze(0)                     # [1, block(q), w, block(k)]
        return a & self.slot_valid[:, None, :, None]

    def dense_mask(self) -> torch.Tensor:
        """The same pattern as a dense ``[seq, seq]`` bool matrix (for checks and for callers that need it)."""
        S, b = self.seq_len, self.block
        q = torch.arange(S).unsqueeze(1)
        k = torch.arange(S).unsqueeze(0)
        return (k <= q) & (k // b > q // b - self.window_blocks)

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, attention_mask: Optional[torch.Tensor] = None):
        B, H, S, D = q.shape
        if S != self.seq_len or D != self.hd:
            raise ValueError(f"expected [..., {self.seq_len}, {self.hd}], got {tuple(q.shape)}")
        b, w = self.block, self.window_blocks
        nb = S // b
        qb = q.reshape(B, H, nb, b, D)
        kb = k.reshape(B, H, nb, b, D)[:, :, self.kv_index]                 # [B, H, nb, w, b, D]
        vb = v.reshape(B, H, nb, b, D)[:, :, self.kv_index]
        scores = torch.einsum("bhnqd,bhnwkd->bhnqwk", qb, kb) * self.scale  # [B, H, nb, b, w, b]
        allow = self.allowed().to(q.device)                                 # [nb, b, w, b]
        if attention_mask is not None:
            am = attention_mask.to(torch.bool).reshape(B, nb, b, nb, b).permute(0, 1, 3, 2, 4)   # [B, nbq, nbk, bq, bk]
            # for every query block, the key blocks of its window: [B, nb, w, bq, bk]
            am = am[:, torch.arange(nb, device=q.device)[:, None], self.kv_index]
            allow = allow.unsqueeze(0) & am.permute(0, 1, 3, 2, 4)
            allow = allow.unsqueeze(1)
        scores = scores.to(self.softmax_dtype).masked_fill(~allow, float("-inf"))
        flat = scores.reshape(B, H, nb, b, w * b)
        probs = torch.softmax(flat, dim=-1)
        probs = torch.nan_to_num(probs, nan=0.0)                            # rows with nothing to attend to
        probs = self.dropout(probs).to(v.dtype).reshape(B, H, nb, b, w, b)
        out = torch.einsum("bhnqwk,bhnwkd->bhnqd", probs, vb)
        return out.reshape(B, H, S, D)


class FixedSparseAttention(nn.Module):
    """Fixed-pattern sparse attention of the Sparse Transformer (reference ``modules/layers.py`` ``FixedSparseAttention``):
    a query attends (causally) to the keys of its own block of ``block_size`` positions and to the last
    ``num_different_global_patterns``-th ... "summary" column group of every earlier block: with ``g`` global patterns,
    head ``h`` uses the ``block_size // g`` columns of slot ``g - 1 - (h % g)`` counted from the end of each block.
    ``q, k, v``: ``[batch, seq, heads * size_per_head]``; ``attention_mask``: ``[batch, seq, seq]`` (1 = may attend).
    Computed densely with the pattern as a mask (the pattern is what the layer defines, not how it is scheduled)."""

    def __init__(self, batch_size=None, num_heads: int = 8, size_per_head: int = 64, block_size: int = 64,
                 seq_length: int = 1024, num_different_global_patterns: int = 4, parallel_config=None):
        super().__init__()
        if seq_length % block_size or block_size % num_different_global_patterns:
            raise ValueError("seq_length must be a multiple of block_size and block_size of num_different_global_patterns")
        self.heads, self.hd, self.block, self.seq, self.g = num_heads, size_per_head, block_size, seq_length, num_different_global_patterns
        pos = torch.arange(seq_length)
        same_block = (pos[:, None] // block_size) == (pos[None, :] // block_size)
        width = block_size // num_different_global_patterns
        masks = []
        for h in range(num_heads):
            slot = num_different_global_patterns - 1 - (h % num_different_global_patterns)
            col = pos % block_size
            summary = (col >= slot * width) & (col < (slot + 1) * width)
            masks.append(same_block | summary[None, :])
        self.register_buffer("pattern", torch.stack(masks) & torch.tril(torch.ones(seq_length, seq_length, dtype=torch.bool)),
                             persistent=False)

    def forward(self, q, k, v, attention_mask=None):
        B, S, _ = q.shape
        qh, kh, vh = (t.view(B, S, self.heads, self.hd).transpose(1, 2).float() for t in (q, k, v))
        scores = qh @ kh.transpose(-1, -2) * self.hd ** -0.5
        allow = self.pattern[None, :, :S, :S].to(q.device)
        if attention_mask is not None:
            allow = allow & attention_mask[:, None].to(torch.bool)
        scores = scores.masked_fill(~allow, float("-inf"))
        probs = torch.nan_to_num(torch.softmax(scores, dim=-1))
        return (probs @ vh).transpose(1, 2).reshape(B, S, self.heads * self.hd).to(q.dtype)
