"""Ring attention: K/V blocks travel around the context-parallel ring while the block at hand is computed.

Reference behaviour: ``training_graph/transformer/flash_attention.py:145-147,167-226`` (the FlashAttention primitive's
ring / send-recv mode), ``mindformers/modules/transformer/transformer.py:537-660`` (hybrid: Ulysses inside a group of
``ulysses_degree_in_cp`` ranks, ring across the groups).

Every rank keeps its own queries and, at step *s*, the K/V block that started *s* positions up the ring. The exchange of
step *s + 1* is posted (``batch_isend_irecv``) before the attention of step *s* starts and awaited after it, so the
transfer runs under the compute; each rank holds two K/V blocks at a time, i.e. memory is O(S / cp), not O(S). Partial
results are merged with their log-sum-exp. The backward pass walks the ring again: each visited block's ``dK`` / ``dV``
accumulate in an fp32 buffer that travels with the block and is home after ``cp`` rotations.

Block attention runs on the flash-attention kernels (forward with log-sum-exp output; backward given the *global*
output and log-sum-exp, which makes the per-block probabilities exact) when the shapes allow it (bf16, head dim 128,
lengths multiples of 128) and on fp32 PyTorch math otherwise (the CPU tests).

Two sequence layouts:

* contiguous: rank r holds tokens ``[r·S, (r+1)·S)``; blocks from later ranks are fully masked and skipped, so the last
  rank works ``cp`` steps and the first one step.
* zig-zag (``cp_zigzag``): the sequence is cut into ``2·cp`` chunks and rank r holds chunks ``r`` and ``2·cp-1-r``. The
  local step is causal over the two chunks; a block from an earlier rank is seen by all local queries but only its
  first chunk is visible; a block from a later rank is seen in full but only by the second local chunk. Every step
  then costs half a block on every rank.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from . import parallel_state as ps


# ---------------------------------------------------------------------------------------------------------------
# block primitives
# ---------------------------------------------------------------------------------------------------------------
def _native_ok(q, k, v) -> bool:
    from ..ops import attention as A
    from ..ops import functional as Fn
    return q.is_cuda and Fn.get_attention_backend() != "sdpa" and A.rect_supported(q, k, v)


def _block_fwd(q, k, v, scale, causal):
    """q ``[B,Sq,H,D]``, k/v ``[B,Sk,Hkv,D]`` → ``(out [B,Sq,H,D] fp32, lse [B,H,Sq] fp32)``; ``causal`` aligns the
    first query with the first key."""
    if _native_ok(q, k, v):
        from ..ops import attention as A
        B, Sq, H, D = q.shape
        o, lse = A.rect_forward(q.contiguous(), k.contiguous(), v.contiguous(), 0, causal, scale)
        return o.view(B, Sq, H, D).float(), lse
    rep = q.shape[2] // k.shape[2]
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        Sq, Sk = q.shape[1], k.shape[1]
        s = s.masked_fill(torch.ones(Sq, Sk, dtype=torch.bool, device=q.device).triu(1), float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    o = torch.matmul(torch.exp(s - lse.unsqueeze(-1)), vf)
    return o.permute(0, 2, 1, 3), lse


def _block_bwd(q, k, v, out, lse, dout, scale, causal):
    """Gradients of one block given the global output ``out [B,Sq,H,D]`` and log-sum-exp ``lse [B,H,Sq]`` of the
    queries: ``(dq [B,Sq,H,D], dk, dv [B,Sk,Hkv,D])`` in fp32."""
    if _native_ok(q, k, v):
        from ..ops import attention as A
        B, Sq, H, D = q.shape
        kc, vc = k.contiguous(), v.contiguous()
        dk, dv = torch.empty_like(kc), torch.empty_like(vc)
        o2 = out.to(torch.bfloat16).reshape(B * Sq, H * D)
        dq = A.rect_backward(q.contiguous(), kc, vc, o2, lse.contiguous(), dout.to(torch.bfloat16).reshape(B * Sq, H * D),
                             dk, dv, 0, causal, scale)
        return dq.float(), dk.float(), dv.float()
    rep = q.shape[2] // k.shape[2]
    do = dout.float().permute(0, 2, 1, 3)
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    delta = (do * out.float().permute(0, 2, 1, 3)).sum(-1)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if causal:
        Sq, Sk = q.shape[1], k.shape[1]
        s = s.masked_fill(torch.ones(Sq, Sk, dtype=torch.bool, device=q.device).triu(1), float("-inf"))
    p = torch.exp(s - lse.unsqueeze(-1))
    dv_b = torch.matmul(p.transpose(-1, -2), do)
    ds = p * (torch.matmul(do, vf.transpose(-1, -2)) - delta.unsqueeze(-1)) * scale
    dq = torch.matmul(ds, kf).permute(0, 2, 1, 3)
    dk_b = torch.matmul(ds.transpose(-1, -2), qf)
    B, H, Sk, D = dk_b.shape
    dk_b = dk_b.view(B, H // rep, rep, Sk, D).sum(2).permute(0, 2, 1, 3)
    dv_b = dv_b.view(B, H // rep, rep, Sk, -1).sum(2).permute(0, 2, 1, 3)
    return dq, dk_b, dv_b


def _merge(out, lse, o_b, lse_b, rows: Optional[slice] = None):
    """Fold a partial result into the running ``(out [B,S,H,D], lse [B,H,S])``; ``rows`` limits it to a query range."""
    if out is None:
        return o_b, lse_b
    if rows is None:
        new = torch.logaddexp(lse, lse_b)
        wa = torch.exp(lse - new).permute(0, 2, 1).unsqueeze(-1)
        wb = torch.exp(lse_b - new).permute(0, 2, 1).unsqueeze(-1)
        return out * wa + o_b * wb, new
    new = torch.logaddexp(lse[:, :, rows], lse_b)
    wa = torch.exp(lse[:, :, rows] - new).permute(0, 2, 1).unsqueeze(-1)
    wb = torch.exp(lse_b - new).permute(0, 2, 1).unsqueeze(-1)
    out[:, rows] = out[:, rows] * wa + o_b * wb          # the running buffers are this function's own
    lse[:, :, rows] = new
    return out, lse


def _plan(step: int, r: int, cp: int, S: int, zigzag: bool):
    """What rank ``r`` computes at ring step ``step`` against the block of rank ``src = (r - step) % cp``:
    ``(query rows, key rows, causal)`` as slices of the local block, or ``None`` when nothing is visible."""
    src = (r - step) % cp
    full = slice(0, S)
    if src == r:
        return full, full, True
    if not zigzag:
        return (full, full, False) if src < r else None
    half = S // 2
    if src < r:
        return full, slice(0, half), False          # an earlier rank: its first chunk lies before both local chunks
    return slice(half, S), full, False              # a later rank: both its chunks lie before the second local chunk


class _Ring:
    """Neighbours of this rank on a ring given by ``ranks`` (global ranks in ring order)."""

    def __init__(self, group, ranks: List[int], index: int):
        self.group, self.ranks, self.r, self.n = group, ranks, index, len(ranks)
        self.next, self.prev = ranks[(index + 1) % self.n], ranks[(index - 1) % self.n]

    def post(self, *bufs):
        """Send every buffer to the next rank and receive its counterpart from the previous one; returns
        ``(requests, received buffers)``."""
        if self.n == 1:
            return [], list(bufs)
        recv = [torch.empty_like(b) for b in bufs]
        ops = []
        for b, rb in zip(bufs, recv):
            ops.append(dist.P2POp(dist.isend, b, self.next, self.group))
            ops.append(dist.P2POp(dist.irecv, rb, self.prev, self.group))
        return dist.batch_isend_irecv(ops), recv


class RingAttnFn(torch.autograd.Function):
    """``forward(q, k, v, scale, ring, zigzag)`` with q/k/v ``[B, S_local, h, d]``."""

    @staticmethod
    def forward(ctx, q, k, v, scale, ring: _Ring, zigzag: bool):
        cp, r, S = ring.n, ring.r, q.shape[1]
        out = lse = None
        kv = torch.stack((k, v)).contiguous()
        for step in range(cp):
            reqs, nxt = ring.post(kv) if step < cp - 1 else ([], [None])
            plan = _plan(step, r, cp, S, zigzag)
            if plan is not None:
                qs, ks, causal = plan
                o_b, lse_b = _block_fwd(q[:, qs], kv[0][:, ks], kv[1][:, ks], scale, causal)
                whole = qs.start == 0 and qs.stop == S
                out, lse = _merge(out, lse, o_b, lse_b, None if whole else qs)
            for q_ in reqs:
                q_.wait()
            if nxt[0] is not None:
                kv = nxt[0]
        ctx.save_for_backward(q, k, v, out.to(q.dtype), lse)
        ctx.scale, ctx.ring, ctx.zigzag = scale, ring, zigzag
        return out.to(q.dtype)

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        scale, ring, zigzag = ctx.scale, ctx.ring, ctx.zigzag
        cp, r, S = ring.n, ring.r, q.shape[1]
        dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        kv = torch.stack((k, v)).contiguous()
        dkv = torch.zeros((2, *k.shape), dtype=torch.float32, device=k.device)
        for step in range(cp):
            # the K/V block for the next step can leave now; its gradient buffer only after this step's contribution
            reqs_kv, nkv = ring.post(kv) if step < cp - 1 else ([], [None])
            plan = _plan(step, r, cp, S, zigzag)
            if plan is not None:
                qs, ks, causal = plan
                dq_b, dk_b, dv_b = _block_bwd(q[:, qs], kv[0][:, ks], kv[1][:, ks], out[:, qs], lse[:, :, qs].contiguous(),
                                              dout[:, qs], scale, causal)
                dq[:, qs] += dq_b
                dkv[0][:, ks] += dk_b
                dkv[1][:, ks] += dv_b
            # after the last step the buffer still has one hop to make to be home
            reqs_g, ndkv = ring.post(dkv)
            for q_ in list(reqs_kv) + list(reqs_g):
                q_.wait()
            dkv = ndkv[0]
            if nkv[0] is not None:
                kv = nkv[0]
        return dq.to(q.dtype), dkv[0].to(k.dtype), dkv[1].to(v.dtype), None, None, None


def ring_attention(q, k, v, scale, group=None, ranks: Optional[List[int]] = None, index: Optional[int] = None,
                   zigzag: bool = False):
    """Causal attention over a sequence split along the ring ``ranks`` (default: the context-parallel group)."""
    if ranks is None:
        group = ps.get_context_parallel_group()
        ranks = ps.get_group_ranks("cp")
        index = ps.get_context_parallel_rank()
    if zigzag and q.shape[1] % 2:
        raise ValueError("the zig-zag layout needs an even number of local tokens")
    return RingAttnFn.apply(q, k, v, scale, _Ring(group, list(ranks), int(index)), bool(zigzag))


def hybrid_attention(q, k, v, scale, ulysses_degree: int):
    """``a2a+p2p``: inside every group of ``ulysses_degree`` consecutive context-parallel ranks the sequence is gathered
    and the heads are scattered (all-to-all), the ring then runs across the groups on ``h / ulysses_degree`` heads, and
    a second all-to-all restores the layout. Ranks hold contiguous sequence chunks."""
    from .context_parallel import _UlyssesA2A
    cp = ps.get_context_parallel_world_size()
    u = int(ulysses_degree)
    if u <= 1:
        return ring_attention(q, k, v, scale)
    if cp % u:
        raise ValueError(f"context parallel size {cp} is not a multiple of ulysses_degree_in_cp {u}")
    if q.shape[2] % u or k.shape[2] % u:
        raise ValueError("the head counts must be divisible by ulysses_degree_in_cp")
    inner_group, _, outer_group, outer_ranks = ps.split_group("cp", u)
    qh, kh, vh = (_UlyssesA2A.apply(t.contiguous(), True, inner_group, u) for t in (q, k, v))
    if cp == u:
        from ..ops import functional as Fn
        o = Fn.attention(qh, kh, vh, causal=True, scale=scale)
    else:
        o = ring_attention(qh, kh, vh, scale, outer_group, outer_ranks, ps.get_context_parallel_rank() // u)
    return _UlyssesA2A.apply(o.contiguous(), False, inner_group, u)
