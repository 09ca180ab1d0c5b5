"""Inference attention of the legacy model stack: cache managers and the attention that uses them.

Reference: ``modules/paged_attention_mgr.py:26-90`` (``PagedAttentionMgr`` owns ``key_cache`` / ``value_cache``
``[num_blocks, block_size, kv_heads, head_dim]`` and wraps ``ReshapeAndCache`` + ``PagedAttention``),
``modules/kvcache_mgr.py`` (``KVCacheMgr``: contiguous ``[batch, kv_heads, seq, head_dim]`` caches written at
``batch_valid_length``) and ``modules/infer_attention.py:66,406-465`` (``InferAttention``: RoPE, cache update,
flash attention for prefill and paged attention for decode, per layer).

The managers are thin owners of cache tensors around the kernels that the parallel-core path uses
(``inference/paged_attention.py``: cache write, split-KV decode attention, flash-attention prefill), so legacy-style
models get the same device code.
"""
from __future__ import annotations

import math
from types import SimpleNamespace
from typing import Optional

import torch
import torch.nn as nn

from ..inference.paged_attention import KVCacheContext, paged_attention_forward
from ..ops import functional as Fn


class PagedAttentionMgr(nn.Module):
    """Block-paged K/V cache of one layer + the two operations on it."""

    def __init__(self, n_heads: int, head_dim: int, n_kv_heads: int, kv_shape, compute_dtype=torch.bfloat16,
                 device=None, scale: Optional[float] = None):
        super().__init__()
        num_blocks, block_size = int(kv_shape[0]), int(kv_shape[1])
        self.n_heads, self.n_kv_heads, self.head_dim = n_heads, n_kv_heads, head_dim
        self.block_size, self.num_blocks = block_size, num_blocks
        self.scale = scale if scale is not None else 1.0 / math.sqrt(head_dim)
        device = device or ("cuda" if torch.cuda.is_available() else "cpu")
        self.ctx = KVCacheContext(1, num_blocks, block_size, n_kv_heads, head_dim, compute_dtype, device)
        self.ctx.layer_offset = 0

    @property
    def key_cache(self) -> torch.Tensor:
        return self.ctx.key_cache[0]

    @property
    def value_cache(self) -> torch.Tensor:
        return self.ctx.value_cache[0]

    def _meta(self, is_prefill, block_tables, slot_mapping, context_lens, q_seq_lens):
        dev = self.key_cache.device
        self.ctx.set_step(is_prefill=is_prefill, block_tables=block_tables, slot_mapping=slot_mapping,
                          context_lens=context_lens, q_seq_lens=q_seq_lens, device=dev)
        return SimpleNamespace(cache=self.ctx)

    def forward(self, query, key, value, slot_mapping, block_tables, batch_valid_length, q_seq_lens=None,
                is_prefill: bool = True) -> torch.Tensor:
        """``query [T, n_heads * hd]``, ``key / value [T, n_kv_heads * hd]`` of the new tokens (flattened batch) →
        ``[T, n_heads * hd]``. ``batch_valid_length`` counts the tokens of every sequence that are in the cache after
        this call; ``q_seq_lens`` the new tokens per sequence (prefill; decode has one each)."""
        T = query.shape[0]
        q = query.view(T, self.n_heads, self.head_dim)
        k = key.view(T, self.n_kv_heads, self.head_dim)
        v = value.view(T, self.n_kv_heads, self.head_dim)
        B = len(batch_valid_length)
        if q_seq_lens is None:
            q_seq_lens = [1] * B if not is_prefill else [int(n) for n in batch_valid_length]
        meta = self._meta(is_prefill, block_tables, slot_mapping, batch_valid_length, q_seq_lens)
        return paged_attention_forward(q, k, v, meta, 1, self.scale)


class KVCacheMgr(nn.Module):
    """Contiguous per-sequence caches ``[batch, kv_heads, max_seq, head_dim]``: prefill writes from position 0, a
    decode step appends one token per sequence at ``batch_valid_length - 1``."""

    def __init__(self, n_kv_heads: int, head_dim: int, max_batch_size: int, max_seq_length: int,
                 compute_dtype=torch.bfloat16, device=None):
        super().__init__()
        device = device or ("cuda" if torch.cuda.is_available() else "cpu")
        shape = (max_batch_size, n_kv_heads, max_seq_length, head_dim)
        self.register_buffer("key_past", torch.zeros(shape, dtype=compute_dtype, device=device), persistent=False)
        self.register_buffer("value_past", torch.zeros(shape, dtype=compute_dtype, device=device), persistent=False)

    def forward(self, key: torch.Tensor, value: torch.Tensor, batch_valid_length: torch.Tensor, is_prefill: bool):
        """``key / value [B, kv_heads, S_new, hd]``. Returns the caches (views over the valid batch rows)."""
        B, _, S, _ = key.shape
        if is_prefill:
            self.key_past[:B, :, :S] = key.to(self.key_past.dtype)
            self.value_past[:B, :, :S] = value.to(self.value_past.dtype)
        else:
            pos = (batch_valid_length.to(key.device).long() - 1).clamp_min(0)
            idx = torch.arange(B, device=key.device)
            self.key_past[idx, :, pos] = key[:, :, 0].to(self.key_past.dtype)
            self.value_past[idx, :, pos] = value[:, :, 0].to(self.value_past.dtype)
        return self.key_past[:B], self.value_past[:B]


class InferAttention(nn.Module):
    """RoPE + cache update + attention for one layer of a legacy-style model.

    ``use_paged_attention=True`` (default): flattened tokens ``[T, heads * hd]`` with block tables and slot mapping.
    Otherwise the contiguous cache: ``[B, S, heads * hd]`` inputs, causal attention over the cached prefix."""

    def __init__(self, n_head: int, head_dim: int, n_kv_head: int, scale_value: Optional[float] = None,
                 block_size: int = 16, num_blocks: int = 512, use_paged_attention: bool = True, max_batch_size: int = 8,
                 max_seq_length: int = 2048, rotary_interleaved: bool = False, compute_dtype=torch.bfloat16, device=None):
        super().__init__()
        self.n_head, self.n_kv_head, self.head_dim = n_head, n_kv_head, head_dim
        self.scale = scale_value if scale_value is not None else 1.0 / math.sqrt(head_dim)
        self.interleaved = rotary_interleaved
        self.paged = use_paged_attention
        if use_paged_attention:
            self.paged_attention_mgr = PagedAttentionMgr(n_head, head_dim, n_kv_head, (num_blocks, block_size),
                                                         compute_dtype, device, self.scale)
        else:
            self.kvcache_mgr = KVCacheMgr(n_kv_head, head_dim, max_batch_size, max_seq_length, compute_dtype, device)

    def _rope(self, x, heads, freqs_cis, positions):
        """``x [T, heads * hd]``; ``freqs_cis = (cos, sin)`` tables ``[max_pos, rot / 2]``."""
        if freqs_cis is None:
            return x
        cos, sin = freqs_cis
        x3 = x.reshape(x.shape[0], heads, self.head_dim).contiguous()
        return Fn.rope(x3, cos, sin, positions, heads, 2 * cos.shape[-1], self.interleaved).reshape(x.shape[0], -1)

    def forward(self, query, key, value, batch_valid_length, block_tables=None, slot_mapping=None, freqs_cis=None,
                positions=None, q_seq_lens=None, is_prefill: bool = True):
        if self.paged:
            T = query.shape[0]
            if freqs_cis is not None and positions is None:
                raise ValueError("positions of the new tokens are needed to apply RoPE")
            q = self._rope(query.view(T, -1), self.n_head, freqs_cis, positions)
            k = self._rope(key.view(T, -1), self.n_kv_head, freqs_cis, positions)
            return self.paged_attention_mgr(q, k, value, slot_mapping, block_tables, batch_valid_length, q_seq_lens,
                                            is_prefill)
        B, S, _ = query.shape
        q = query.view(B, S, self.n_head, self.head_dim)
        k = key.view(B, S, self.n_kv_head, self.head_dim)
        v = value.view(B, S, self.n_kv_head, self.head_dim)
        if freqs_cis is not None:
            pos = positions if positions is not None else torch.arange(S, device=query.device).repeat(B)
            q = self._rope(q.reshape(B * S, -1), self.n_head, freqs_cis, pos).view(B, S, self.n_head, self.head_dim)
            k = self._rope(k.reshape(B * S, -1), self.n_kv_head, freqs_cis, pos).view(B, S, self.n_kv_head, self.head_dim)
        kc, vc = self.kvcache_mgr(k.transpose(1, 2), v.transpose(1, 2), batch_valid_length, is_prefill)
        if is_prefill:
            out = Fn.attention(q, k, v, causal=True, scale=self.scale)
            return out.reshape(B, S, -1)
        outs = []
        for b in range(B):
            n = int(batch_valid_length[b])
            kk, vv = kc[b, :, :n].transpose(0, 1).unsqueeze(0), vc[b, :, :n].transpose(0, 1).unsqueeze(0)
            outs.append(Fn.attention_reference(q[b:b + 1], kk, vv, causal=False, scale=self.scale))
        return torch.cat(outs, dim=0).reshape(B, S, -1)
