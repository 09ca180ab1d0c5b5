"""Context-parallel attention: all-gather KV, ring (P2P) exchange, Ulysses all-to-all; packed-sequence attention.

Reference: the reference toggles these inside its FlashAttention primitive
(``training_graph/transformer/flash_attention.py:145-147,167-226`` for ring / all-gather layouts,
``attention.py:203-222,360-428`` for the Ulysses transposes). Here the mechanisms are explicit:

* ``all_gather``: K/V of all ranks are gathered, each rank attends its query chunk (zig-zag balanced).
* ``p2p`` (ring): K/V blocks rotate around the ring while the local block computes; partial outputs are
  merged with their log-sum-exp.
* ``a2a`` (Ulysses): sequence ↔ head all-to-all around a full-sequence attention.
* ``a2a+p2p`` (hybrid): Ulysses inside groups of ``ulysses_degree_in_cp`` ranks, the ring across the groups.

The ring and the hybrid live in ``ring_attention.py``. On a GPU ``p2p`` and ``all_gather`` take the fused peer-memory
path (K/V pulled by peer loads into one buffer, O(S) memory) unless ``fused_cp_comm`` is off.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from ..ops import functional as Fn
from . import mappings as M
from . import parallel_state as ps


def varlen_attention(q, k, v, cu_seqlens, scale):
    """Causal attention over packed sequences: tokens attend within their own segment only.
    q/k/v: [B, S, h, d]; ``cu_seqlens``: cumulative boundaries over the flattened B*S tokens."""
    B, S = q.shape[:2]
    T = B * S
    qf, kf, vf = (t.reshape(1, T, t.shape[2], t.shape[3]) for t in (q, k, v))
    bounds = cu_seqlens.tolist()
    outs = []
    for a, b in zip(bounds[:-1], bounds[1:]):
        if b > a:
            outs.append(Fn.attention(qf[:, a:b], kf[:, a:b], vf[:, a:b], causal=True, scale=scale))
    return torch.cat(outs, dim=1).reshape(B, S, q.shape[2], v.shape[3])


def _attn_with_lse(q, k, v, scale, causal, q_offset=0):
    """Reference-math attention that also returns the log-sum-exp; used by the ring merge."""
    B, Sq, Hq, D = q.shape
    rep = Hq // k.shape[2]
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        qi = torch.arange(Sq, device=q.device).unsqueeze(-1) + q_offset
        ki = torch.arange(k.shape[1], device=q.device).unsqueeze(0)
        s = s.masked_fill(ki > qi, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    o = torch.matmul(p, vf)
    return o.permute(0, 2, 1, 3), lse.permute(0, 2, 1)  # [B,S,H,D], [B,S,H]


class _UlyssesA2A(torch.autograd.Function):
    """[B, S/cp, h, d] ↔ [B, S, h/cp, d] all-to-all; ``to_heads`` picks the direction."""
    @staticmethod
    def forward(ctx, x, to_heads, group, cp):
        ctx.to_heads, ctx.group, ctx.cp = to_heads, group, cp
        B, S, h, d = x.shape
        if to_heads:
            xs = x.reshape(B, S, cp, h // cp, d).permute(2, 0, 1, 3, 4).contiguous()
            out = torch.empty_like(xs)
            dist.all_to_all_single(out, xs, group=group)
            return out.permute(1, 0, 2, 3, 4).reshape(B, cp * S, h // cp, d)
        xs = x.reshape(B, cp, S // cp, h, d).permute(1, 0, 2, 3, 4).contiguous()
        out = torch.empty_like(xs)
        dist.all_to_all_single(out, xs, group=group)
        return out.permute(1, 2, 0, 3, 4).reshape(B, S // cp, cp * h, d)

    @staticmethod
    def backward(ctx, g):
        return _UlyssesA2A.apply(g.contiguous(), not ctx.to_heads, ctx.group, ctx.cp), None, None, None


def ulysses_attention(q, k, v, scale, group=None):
    group = group if group is not None else ps.get_context_parallel_group()
    cp = ps.get_context_parallel_world_size()
    if q.shape[2] % cp or k.shape[2] % cp:
        raise ValueError("Ulysses context parallelism needs head counts divisible by the cp size")
    qh, kh, vh = (_UlyssesA2A.apply(t.contiguous(), True, group, cp) for t in (q, k, v))
    o = Fn.attention(qh, kh, vh, causal=True, scale=scale)
    return _UlyssesA2A.apply(o.contiguous(), False, group, cp)


class _AllGatherSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, cp):
        ctx.group, ctx.cp = group, cp
        parts = [torch.empty_like(x) for _ in range(cp)]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.cat(parts, dim=1)

    @staticmethod
    def backward(ctx, g):
        cp = ctx.cp
        chunks = [c.contiguous() for c in g.chunk(cp, dim=1)]
        out = torch.empty_like(chunks[0])
        dist.reduce_scatter(out, chunks, group=ctx.group)
        return out, None, None


def allgather_kv_attention(q, k, v, scale, group=None):
    """Gather K/V over the cp group; this rank's queries (tokens [r*S,(r+1)*S)) attend the prefix."""
    group = group if group is not None else ps.get_context_parallel_group()
    cp = ps.get_context_parallel_world_size()
    r = ps.get_context_parallel_rank()
    kf = _AllGatherSeq.apply(k, group, cp)
    vf = _AllGatherSeq.apply(v, group, cp)
    S = q.shape[1]
    end = (r + 1) * S
    if q.is_cuda:
        o, _ = _attn_with_lse(q, kf[:, :end], vf[:, :end], scale, causal=True, q_offset=r * S)
        return o.to(q.dtype)
    return Fn.attention_reference(q, kf[:, :end], vf[:, :end], True, scale, q_offset=r * S)


def context_parallel_attention(q, k, v, scale, config):
    kind = config.cp_comm_type
    if kind in ("p2p", "all_gather") and getattr(config, "fused_cp_comm", True) and q.is_cuda:
        from . import fused_comm, fused_cp
        if fused_comm.cp_enabled() and fused_cp.supported(q, k, v):
            # K/V exchange by peer loads + rectangular flash attention (same result as the ring)
            return fused_cp.fused_cp_attention(q, k, v, scale, zigzag=bool(getattr(config, "cp_zigzag", False)))
    if kind == "p2p":
        # K/V blocks travel the ring under the compute, memory O(S / cp); zig-zag balances the causal work
        from .ring_attention import ring_attention
        return ring_attention(q, k, v, scale, zigzag=bool(getattr(config, "cp_zigzag", False)))
    if kind == "a2a":
        return ulysses_attention(q, k, v, scale)
    if kind == "a2a+p2p":
        from .ring_attention import hybrid_attention
        if getattr(config, "cp_zigzag", False):
            raise ValueError("a2a+p2p context parallelism uses contiguous sequence chunks: switch cp_zigzag off")
        u = int(getattr(config, "ulysses_degree_in_cp", 0) or 0)
        sizes = getattr(config, "hierarchical_context_parallel_sizes", None)
        if not u and sizes:
            u = int(sizes[0])
        return hybrid_attention(q, k, v, scale, u or 1)
    if kind == "all_gather":
        return allgather_kv_attention(q, k, v, scale)
    raise NotImplementedError(f"cp_comm_type {kind!r}")
