"""Attention over the paged KV cache: cache allocation, prefill and decode paths.

Reference: ``parallel_core/inference/transformer/flash_attention.py`` (prefill = cache write + varlen flash
attention :94-107; decode = paged attention :109-145), MLA mode with one latent "head" of width
``kv_lora_rank + rope_dim`` (``multi_latent_attention.py:401-448``), cache shapes from
``generation/text_generator.py:114-160``.

``KVCacheContext`` travels in ``AttnMeta.cache``; it owns the per-layer cache tensors and the device copies of
the block table, slot mapping and lengths for the current step.
"""
from __future__ import annotations

import os

import math
from typing import List, Optional

import torch

from ..ops import _lib
from ..ops import functional as Fn


class KVCacheContext:
    """Per-layer paged caches ``[num_blocks, block_size, kv_heads, head_dim]`` (or the 576-wide latent cache of
    multi-latent attention) plus the metadata of the current step: block tables, slot mapping, context lengths, new
    tokens per sequence."""

    def __init__(self, num_layers: int, num_blocks: int, block_size: int, kv_heads: int, head_dim: int,
                 dtype=torch.bfloat16, device="cuda", mla_latent_dim: Optional[int] = None,
                 kv_cache_dtype: Optional[str] = None):
        """``kv_cache_dtype="int8"`` stores keys and values as int8 codes with one fp32 scale per token and KV head
        (``key_scale`` / ``value_scale`` ``[num_blocks, block_size, kv_heads]``): half the bytes per cached token, read
        back by the decode kernel and by prefill with history. Not available for the multi-latent cache."""
        self.num_layers, self.num_blocks, self.block_size = num_layers, num_blocks, block_size
        self.kv_heads, self.head_dim, self.mla_dim = kv_heads, head_dim, mla_latent_dim
        self.int8 = str(kv_cache_dtype or "").lower() in ("int8", "torch.int8")
        self.key_scale = self.value_scale = None
        self.compute_dtype = dtype
        if self.int8 and mla_latent_dim:
            raise ValueError("an int8 KV cache is not available for multi-latent attention")
        if self.int8:
            shape = (num_blocks, block_size, kv_heads, head_dim)
            self.key_cache = [torch.zeros(shape, dtype=torch.int8, device=device) for _ in range(num_layers)]
            self.value_cache = [torch.zeros(shape, dtype=torch.int8, device=device) for _ in range(num_layers)]
            self.key_scale = [torch.ones(shape[:3], dtype=torch.float32, device=device) for _ in range(num_layers)]
            self.value_scale = [torch.ones(shape[:3], dtype=torch.float32, device=device) for _ in range(num_layers)]
        elif mla_latent_dim:
            self.key_cache = [torch.zeros(num_blocks, block_size, 1, mla_latent_dim, dtype=dtype, device=device)
                              for _ in range(num_layers)]
            self.value_cache = [None] * num_layers
        else:
            shape = (num_blocks, block_size, kv_heads, head_dim)
            self.key_cache = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(num_layers)]
            self.value_cache = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(num_layers)]
        self.is_prefill = True
        self.block_tables = None      # int32 [B, max_blocks]
        self.slot_mapping = None      # int32 [T]
        self.context_lens = None      # int32 [B] tokens in cache after this step
        self.q_seq_lens = None        # int32 [B] new tokens of each sequence in this step
        self.last_token_index = None  # int64 [B] row of the last new token of each sequence
        self.cu_q = None              # python list of cumulative q lengths
        self.layer_offset = 0

    def set_step(self, *, is_prefill, block_tables, slot_mapping, context_lens, q_seq_lens, device):
        self.is_prefill = is_prefill
        self.block_tables = torch.as_tensor(block_tables, dtype=torch.int32, device=device).contiguous()
        self.slot_mapping = torch.as_tensor(slot_mapping, dtype=torch.int32, device=device).contiguous()
        self.context_lens = torch.as_tensor(context_lens, dtype=torch.int32, device=device).contiguous()
        q = [int(x) for x in q_seq_lens]
        self.q_seq_lens = torch.as_tensor(q, dtype=torch.int32, device=device)
        cu = [0]
        for n in q:
            cu.append(cu[-1] + n)
        self.cu_q = cu
        # sequences without new tokens in this step (finished prompts of a chunked prefill, idle serving slots) have
        # no row of their own: one entry per sequence that has tokens
        self.last_token_index = torch.as_tensor([c - 1 for c, n in zip(cu[1:], q) if n > 0], dtype=torch.int64,
                                                device=device)


def _write_cache(cache: KVCacheContext, layer: int, k: torch.Tensor, v: Optional[torch.Tensor]):
    """k, v: [T, heads, hd] (views with token stride); scatter rows into the layer's cache by slot."""
    T = k.shape[0]
    kc, vc = cache.key_cache[layer], cache.value_cache[layer]
    row = k.shape[1] * k.shape[2]
    if getattr(cache, "int8", False):
        ks, vs = cache.key_scale[layer], cache.value_scale[layer]
        if k.is_cuda and k.dtype == torch.bfloat16 and k.stride(2) == 1 and k.stride(1) == k.shape[2] \
                and v.stride(2) == 1 and v.stride(1) == v.shape[2]:
            rc = _lib.get_lib().mfb_reshape_and_cache_int8(
                k.data_ptr(), v.data_ptr(), kc.data_ptr(), vc.data_ptr(), ks.data_ptr(), vs.data_ptr(),
                cache.slot_mapping.data_ptr(), T, k.shape[1], k.shape[2], k.stride(0), v.stride(0), _lib.stream_ptr())
            _lib.check(rc, "mfb_reshape_and_cache_int8")
            _lib.count_launch()
            return
        slots = cache.slot_mapping.long()
        ok = slots >= 0
        for src, dst, sc in ((k, kc, ks), (v, vc, vs)):
            x = src.reshape(T, src.shape[1], src.shape[2])[ok].float()
            amax = x.abs().amax(-1)
            scale = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax))
            q = torch.round(x / scale.unsqueeze(-1)).clamp(-127, 127).to(torch.int8)
            dst.view(-1, src.shape[1], src.shape[2])[slots[ok]] = q
            sc.view(-1, src.shape[1])[slots[ok]] = scale
        return
    if k.is_cuda and k.dtype == torch.bfloat16 and row % 8 == 0 and k.stride(2) == 1 and k.stride(1) == k.shape[2]:
        rc = _lib.get_lib().mfb_reshape_and_cache(k.data_ptr(), _lib.ptr(v), kc.data_ptr(), _lib.ptr(vc),
                                                  cache.slot_mapping.data_ptr(), T, row, k.stride(0),
                                                  v.stride(0) if v is not None else 0, _lib.stream_ptr())
        _lib.check(rc, "mfb_reshape_and_cache")
        _lib.count_launch()
        return
    slots = cache.slot_mapping.long()
    ok = slots >= 0
    kc.view(-1, row)[slots[ok]] = k.reshape(T, row)[ok].to(kc.dtype)
    if v is not None:
        vc.view(-1, row)[slots[ok]] = v.reshape(T, row)[ok].to(vc.dtype)


def _gather(cache_t: torch.Tensor, table_row: torch.Tensor, n: int, block_size: int,
            scale_t: Optional[torch.Tensor] = None, dtype=None) -> torch.Tensor:
    """The first ``n`` cached rows of one sequence as a contiguous tensor (de-quantised when ``scale_t`` is given)."""
    nb = -(-n // block_size)
    blocks = table_row[:nb].long()
    rows = cache_t[blocks].reshape(nb * block_size, *cache_t.shape[2:])[:n]
    if scale_t is not None:
        sc = scale_t[blocks].reshape(nb * block_size, -1)[:n]
        rows = (rows.float() * sc.unsqueeze(-1)).to(dtype or torch.bfloat16)
    return rows


def _layer_scales(cache, layer):
    if getattr(cache, "int8", False):
        return cache.key_scale[layer], cache.value_scale[layer]
    return None, None


# Decode attention over a bf16 cache with head dim 128 runs on the tensor cores (``paged_decode_tc.cu``);
# ``MFB_PAGED_DECODE=cuda_core`` (or ``set_paged_decode_kernel``) keeps the split-KV kernel on the CUDA cores, which also
# serves head dim 64 and the int8 cache.
_DECODE_KERNEL = "cuda_core" if os.environ.get("MFB_PAGED_DECODE", "tensor_core") == "cuda_core" else "tensor_core"


def set_paged_decode_kernel(kind: str) -> None:
    global _DECODE_KERNEL
    if kind not in ("tensor_core", "cuda_core"):
        raise ValueError("kind must be 'tensor_core' or 'cuda_core'")
    _DECODE_KERNEL = kind


def paged_attention_forward(q, k, v, meta, layer_number: int, scale: float):
    """q: [T, nq, hd]; k/v: [T, nkv, hd] of the new tokens. Returns [T, nq*hd]."""
    cache: KVCacheContext = meta.cache
    layer = layer_number - 1 - cache.layer_offset
    _write_cache(cache, layer, k, v)
    T, nq, hd = q.shape
    nkv = k.shape[1]
    B = cache.context_lens.shape[0]
    if not cache.is_prefill and T == B:
        out = torch.empty((T, nq, hd), dtype=q.dtype, device=q.device)
        if q.is_cuda and q.dtype == torch.bfloat16 and hd in (64, 128) and nq // nkv <= 16:
            qc = q.contiguous()
            lib = _lib.get_lib()
            max_blocks = cache.block_tables.shape[1]
            ksc, vsc = _layer_scales(cache, layer)
            if ksc is None and _DECODE_KERNEL == "tensor_core" \
                    and lib.mfb_paged_decode_tc_supported(nq, nkv, hd, cache.block_size):
                # bf16 cache, head dim 128: Q K^T and P V on the tensor cores, K / V tiles streamed by TMA
                splits = lib.mfb_paged_decode_tc_splits(B, nkv, max_blocks * cache.block_size)
                need = lib.mfb_paged_decode_scratch_bytes(B, nq, hd, splits)
                scratch = getattr(cache, "_decode_scratch", None)
                if scratch is None or scratch.numel() * 4 < need:
                    scratch = cache._decode_scratch = torch.empty((need + 3) // 4, dtype=torch.float32, device=q.device)
                kc = cache.key_cache[layer]
                rc = lib.mfb_paged_decode_attention_tc(
                    qc.data_ptr(), kc.data_ptr(), cache.value_cache[layer].data_ptr(), cache.block_tables.data_ptr(),
                    cache.context_lens.data_ptr(), out.data_ptr(), scratch.data_ptr(), splits, B, nq, nkv, kc.shape[0],
                    cache.block_size, max_blocks, float(scale), _lib.status_word(q.device).data_ptr(), _lib.stream_ptr())
                _lib.check(rc, "mfb_paged_decode_attention_tc")
                _lib.count_launch(2)
                return out.view(T, nq * hd)
            splits = lib.mfb_paged_decode_splits(B, nkv, cache.block_size, max_blocks)
            need = lib.mfb_paged_decode_scratch_bytes(B, nq, hd, splits)
            scratch = getattr(cache, "_decode_scratch", None)
            if scratch is None or scratch.numel() * 4 < need:
                scratch = cache._decode_scratch = torch.empty((need + 3) // 4, dtype=torch.float32, device=q.device)
            rc = lib.mfb_paged_decode_attention_ex(
                qc.data_ptr(), cache.key_cache[layer].data_ptr(), cache.value_cache[layer].data_ptr(),
                _lib.ptr(ksc), _lib.ptr(vsc),
                cache.block_tables.data_ptr(), cache.context_lens.data_ptr(), out.data_ptr(), scratch.data_ptr(), splits,
                B, nq, nkv, hd, cache.block_size, max_blocks, float(scale), _lib.stream_ptr())
            _lib.check(rc, "mfb_paged_decode_attention_ex")
            _lib.count_launch(2)
            return out.view(T, nq * hd)
        lens = cache.context_lens.tolist()
        ksc, vsc = _layer_scales(cache, layer)
        for b in range(B):
            kk = _gather(cache.key_cache[layer], cache.block_tables[b], lens[b], cache.block_size, ksc, q.dtype)
            vv = _gather(cache.value_cache[layer], cache.block_tables[b], lens[b], cache.block_size, vsc, q.dtype)
            o = Fn.attention_reference(q[b:b + 1].unsqueeze(0), kk.unsqueeze(0), vv.unsqueeze(0), causal=False, scale=scale)
            out[b] = o[0, 0]
        return out.view(T, nq * hd)
    # prefill (optionally with history, e.g. chunked prefill): per-sequence causal attention
    outs = []
    lens = cache.context_lens.tolist()
    for b in range(B):
        a, e = cache.cu_q[b], cache.cu_q[b + 1]
        if e == a:
            continue
        nq_tok = e - a
        if lens[b] == nq_tok:
            o = Fn.attention(q[a:e].unsqueeze(0), k[a:e].unsqueeze(0), v[a:e].unsqueeze(0), causal=True, scale=scale)
        else:
            ksc, vsc = _layer_scales(cache, layer)
            kk = _gather(cache.key_cache[layer], cache.block_tables[b], lens[b], cache.block_size, ksc, q.dtype)
            vv = _gather(cache.value_cache[layer], cache.block_tables[b], lens[b], cache.block_size, vsc, q.dtype)
            o = Fn.attention_reference(q[a:e].unsqueeze(0), kk.unsqueeze(0), vv.unsqueeze(0), causal=True, scale=scale,
                                       q_offset=lens[b] - nq_tok)
        outs.append(o.reshape(nq_tok, nq * v.shape[-1]))
    return torch.cat(outs, dim=0)


def set_mla_decode_variant(variant: str) -> None:
    """Choose the MLA decode kernel: ``"single"`` (one CTA per work item, ``ops/csrc/mla_decode.cu``) or ``"cluster"``
    (two CTAs of a cluster split the latent columns and read the cache once, ``ops/csrc/mla_decode_cluster.cu``)."""
    if variant not in ("single", "cluster"):
        raise ValueError(f"unknown MLA decode variant {variant!r}")
    _lib.get_lib().mfb_mla_decode_set_variant(1 if variant == "cluster" else 0)


def mla_decode_attention(q_cat: torch.Tensor, latent_cache: torch.Tensor, block_tables: torch.Tensor,
                         context_lens: torch.Tensor, block_size: int, scale: float, holder=None) -> torch.Tensor:
    """``q_cat [B, heads, 576]`` (absorbed query ‖ rope query) against the paged latent cache
    ``[num_blocks, block_size, (1,) 576]`` → latent-space output ``[B, heads, 512]``; ``context_lens`` counts the
    tokens in the cache, the current one included. ``holder`` keeps the scratch buffer between calls."""
    B, nh, dim = q_cat.shape
    if dim != 576 or q_cat.dtype != torch.bfloat16 or latent_cache.dtype != torch.bfloat16:
        raise ValueError("mla_decode_attention: bf16 tensors with a latent width of 512 + 64 are required")
    lib = _lib.get_lib()
    max_blocks = block_tables.shape[1]
    splits = lib.mfb_mla_decode_splits(B, nh, max_blocks * block_size)
    need = lib.mfb_mla_decode_scratch_bytes(B, nh, splits)
    scratch = getattr(holder, "_mla_scratch", None) if holder is not None else None
    if scratch is None or scratch.numel() * 4 < need:
        scratch = torch.empty((need + 3) // 4, dtype=torch.float32, device=q_cat.device)
        if holder is not None:
            holder._mla_scratch = scratch
    out = torch.empty((B, nh, 512), dtype=torch.bfloat16, device=q_cat.device)
    num_blocks = latent_cache.shape[0]
    rc = lib.mfb_mla_decode_attention(q_cat.data_ptr(), latent_cache.data_ptr(), block_tables.data_ptr(),
                                      context_lens.data_ptr(), out.data_ptr(), scratch.data_ptr(), splits, B, nh,
                                      num_blocks, block_size, max_blocks, float(scale),
                                      _lib.status_word(q_cat.device).data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "mfb_mla_decode_attention")
    _lib.count_launch(2)
    return out


def mla_paged_attention_forward(attn, q_nope, q_pe, kv_c, k_pe, meta):
    """Multi-latent attention with a latent cache ``[kv_lora ‖ k_pe]``.

    Prefill expands K/V from the latent with ``linear_kvb``; decode absorbs the up-projections: queries are
    mapped into the latent space (``q_nope @ W_UK``), attention runs against the cached latents, and the result is
    mapped back with ``W_UV`` (reference ``multi_latent_attention.py:219-231,434-448``).
    """
    cache: KVCacheContext = meta.cache
    layer = attn.layer_number - 1 - cache.layer_offset
    T = q_nope.shape[0]
    latent = torch.cat((kv_c, k_pe.reshape(T, -1)), dim=-1).unsqueeze(1)     # [T, 1, rank + rope]
    _write_cache(cache, layer, latent.contiguous(), None)
    nh, nope, rope_d, vd, rank = attn.nh, attn.nope, attn.rope_d, attn.vd, attn.kv_rank
    w = attn.linear_kvb.weight.view(nh, nope + vd, rank)
    w_uk, w_uv = w[:, :nope], w[:, nope:]                                      # [nh, nope, rank], [nh, vd, rank]
    B = cache.context_lens.shape[0]
    if (not cache.is_prefill and T == B and q_nope.is_cuda and q_nope.dtype == torch.bfloat16 and rank == 512
            and rope_d == 64 and cache.block_size in (16, 32, 64, 128)):
        # decode: absorbed queries against the latent cache in one tcgen05 kernel (ops/csrc/mla_decode.cu)
        q_lat = torch.einsum("bhn,hnr->bhr", q_nope, w_uk)
        q_cat = torch.cat((q_lat, q_pe.reshape(B, nh, rope_d)), dim=-1).contiguous()
        o_lat = mla_decode_attention(q_cat, cache.key_cache[layer], cache.block_tables, cache.context_lens,
                                     cache.block_size, attn.scale, cache)
        return torch.einsum("bhr,hvr->bhv", o_lat, w_uv).reshape(B, nh * vd)
    lens = cache.context_lens.tolist()
    q_lens = [cache.cu_q[b + 1] - cache.cu_q[b] for b in range(B)]
    if (cache.is_prefill and q_nope.is_cuda and q_nope.dtype == torch.bfloat16 and nope == 128 and rope_d == 64
            and vd == 128 and all(ql == n and ql % 128 == 0 and ql > 0 for ql, n in zip(q_lens, lens))):
        # prefill without history: expand K / V from the latents and run the flash-attention kernel (192 / 128 heads)
        from ..ops import attention as native
        kv = attn._col_nosp(attn.linear_kvb, kv_c).view(T, nh, nope + vd)
        k = torch.cat((kv[..., :nope], k_pe.reshape(T, 1, rope_d).expand(T, nh, rope_d)), dim=-1)
        v = kv[..., nope:]
        qf = torch.cat((q_nope, q_pe), dim=-1)
        if len(set(q_lens)) == 1:
            S = q_lens[0]
            o = native.mla_forward(qf.view(B, S, nh, -1), k.view(B, S, nh, -1), v.reshape(B, S, nh, vd), True, attn.scale)
            return o.reshape(T, nh * vd)
        outs = []
        for b in range(B):
            a, e = cache.cu_q[b], cache.cu_q[b + 1]
            o = native.mla_forward(qf[a:e].unsqueeze(0), k[a:e].unsqueeze(0), v[a:e].unsqueeze(0), True, attn.scale)
            outs.append(o.reshape(e - a, nh * vd))
        return torch.cat(outs, dim=0)
    outs = []
    for b in range(B):
        a, e = cache.cu_q[b], cache.cu_q[b + 1]
        if e == a:
            continue
        lat = _gather(cache.key_cache[layer], cache.block_tables[b], lens[b], cache.block_size)[:, 0]  # [L, rank+rope]
        c, pe = lat[:, :rank].float(), lat[:, rank:].float()
        q_lat = torch.einsum("thn,hnr->thr", q_nope[a:e].float(), w_uk.float())    # absorbed query
        s = (torch.einsum("thr,lr->htl", q_lat, c) + torch.einsum("thd,ld->htl", q_pe[a:e].float(), pe)) * attn.scale
        nq_tok, L = e - a, lens[b]
        qi = torch.arange(nq_tok, device=s.device).unsqueeze(-1) + (L - nq_tok)
        ki = torch.arange(L, device=s.device).unsqueeze(0)
        s = s.masked_fill((ki > qi).unsqueeze(0), float("-inf"))
        p = torch.softmax(s, dim=-1)
        o_lat = torch.einsum("htl,lr->thr", p, c)
        o = torch.einsum("thr,hvr->thv", o_lat, w_uv.float())
        outs.append(o.reshape(nq_tok, nh * vd).to(q_nope.dtype))
    return torch.cat(outs, dim=0)
