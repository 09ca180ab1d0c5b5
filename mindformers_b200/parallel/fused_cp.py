"""Context-parallel attention on the peer-memory K/V exchange kernels (``ops/csrc/cp_comm.cu``) and the
rectangular flash-attention kernels.

Forward: K and V of this rank's chunk go to a peer-mapped staging buffer; ``cp_gather`` pulls every rank's chunk
into a local full-sequence K / V (natural token order), then the local queries attend with the causal diagonal at
their global position. Backward: K / V are gathered again (cheaper than keeping ``cp`` full copies per layer), the
attention backward writes partial dK / dV for the whole sequence into a peer-mapped buffer, and
``cp_reduce_scatter`` sums every rank's partials for this rank's chunk.

With ``zigzag`` the sequence is cut into ``2·cp`` chunks and rank ``r`` owns chunks ``r`` and ``2·cp−1−r`` (its
local tokens are those two chunks concatenated), which evens out the causal work: every rank then runs two
rectangular attentions of half the local length.

The reference asks MindSpore for ring attention with two primitive attributes
(``training_graph/transformer/flash_attention.py:145-147``); the exchanged bytes are the same, here they move by
peer loads issued from this library's kernels instead of send/recv pairs.
"""
from __future__ import annotations

import ctypes
from typing import Dict

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import attention as A
from . import parallel_state as ps
from . import symm_mem


class CPExchange:
    """Peer-memory state of the context-parallel K/V exchange of one group: symmetric K/V and dK/dV buffers, flag words,
    epoch counter."""

    _instances: Dict[tuple, "CPExchange"] = {}

    @classmethod
    def get(cls, s_local: int, width: int) -> "CPExchange":
        grp = ps.get_context_parallel_group()
        key = (id(grp), s_local, width)
        inst = cls._instances.get(key)
        if inst is None:
            inst = cls._instances[key] = cls(grp, s_local, width)
        return inst

    def __init__(self, group, s_local: int, width: int):
        self.group = group
        self.world = ps.get_context_parallel_world_size()
        self.rank = ps.get_context_parallel_rank()
        self.s_local, self.width = s_local, width
        self.dev = torch.device("cuda", torch.cuda.current_device())
        self.lib = _lib.get_lib()
        self.epoch = 0
        arr = ctypes.c_longlong * self.world
        n_stage = 2 * s_local * width
        n_full = n_stage * self.world
        tag = f"{id(group)}.{s_local}.{width}"
        if self.world > 1:
            stage = symm_mem.allocate(f"cp.stage.{tag}", n_stage * 2, group, self.dev)
            dfull = symm_mem.allocate(f"cp.dfull.{tag}", n_full * 2, group, self.dev)
            flags = symm_mem.allocate(f"cp.flags.{tag}", self.lib.mfb_cp_flag_words() * 4, group, self.dev)
            flags.tensor.zero_()
            self.stage = stage.tensor.view(torch.bfloat16)[:n_stage].view(2, s_local, width)
            self.dfull = dfull.tensor.view(torch.bfloat16)[:n_full].view(2, s_local * self.world, width)
            self.peer_stage, self.peer_dfull = arr(*stage.ptrs), arr(*dfull.ptrs)
            self.peer_flags = arr(*flags.ptrs)
            self._keep = (stage, dfull, flags)
            torch.cuda.synchronize()
            dist.barrier(group=group)
        else:
            self.stage = torch.empty(2, s_local, width, dtype=torch.bfloat16, device=self.dev)
            self.dfull = torch.empty(2, s_local, width, dtype=torch.bfloat16, device=self.dev)
            self.peer_stage, self.peer_dfull = arr(self.stage.data_ptr()), arr(self.dfull.data_ptr())
            self.peer_flags = None

    def _status(self):
        return _lib.status_word(self.dev).data_ptr()

    def _next(self):
        self.epoch += 1
        return self.epoch

    def gather(self, k: torch.Tensor, v: torch.Tensor, zigzag: bool) -> torch.Tensor:
        """k, v ``[S_local, W]`` → full ``[2, S_total, W]`` (a fresh local tensor)."""
        self.stage[0].copy_(k)
        self.stage[1].copy_(v)
        full = torch.empty(2, self.s_local * self.world, self.width, dtype=torch.bfloat16, device=self.dev)
        rc = self.lib.mfb_cp_gather(self.world, self.rank, self._next(), 0, int(zigzag), self.s_local, self.width,
                                    self.peer_stage, self.peer_flags, full.data_ptr(), self._status(), _lib.stream_ptr())
        _lib.check(rc, "mfb_cp_gather")
        self.barrier(1)       # every rank has finished reading the staging buffers
        _lib.count_launch(1)
        return full

    def reduce_scatter(self, zigzag: bool) -> torch.Tensor:
        """Sum of all ranks' ``dfull`` over this rank's rows → ``[2, S_local, W]``."""
        out = torch.empty(2, self.s_local, self.width, dtype=torch.bfloat16, device=self.dev)
        rc = self.lib.mfb_cp_reduce_scatter(self.world, self.rank, self._next(), 2, int(zigzag), self.s_local, self.width,
                                            self.peer_dfull, self.peer_flags, out.data_ptr(), self._status(),
                                            _lib.stream_ptr())
        _lib.check(rc, "mfb_cp_reduce_scatter")
        self.barrier(3)       # every rank has finished reading the partial-gradient buffers
        _lib.count_launch(1)
        return out

    def barrier(self, phase: int):
        if self.world > 1:
            rc = self.lib.mfb_cp_barrier(self.world, self.rank, self._next(), phase, self.peer_flags, self._status(),
                                         _lib.stream_ptr())
            _lib.check(rc, "mfb_cp_barrier")
            _lib.count_launch(1)


def _segments(rank: int, world: int, s_local: int, zigzag: bool):
    """``[(local_begin, local_end, global_offset)]`` of this rank's query chunks."""
    if not zigzag:
        return [(0, s_local, rank * s_local)]
    h = s_local // 2
    return [(0, h, rank * h), (h, s_local, (2 * world - 1 - rank) * h)]


class _FusedCPAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, zigzag):
        # q [1, S, nq, 128]; k, v [1, S, nkv, 128]
        _, S, nq, hd = q.shape
        nkv = k.shape[2]
        W = nkv * hd
        ex = CPExchange.get(S, W)
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        full = ex.gather(k.view(S, W), v.view(S, W), zigzag)
        St = S * ex.world
        kf, vf = full[0].view(1, St, nkv, hd), full[1].view(1, St, nkv, hd)
        outs, lses = [], []
        for a, b, off in _segments(ex.rank, ex.world, S, zigzag):
            kend = off + (b - a)                              # keys beyond the diagonal are never read
            o, lse = A.rect_forward(q[:, a:b], kf[:, :kend], vf[:, :kend], off, True, scale)
            outs.append(o)
            lses.append(lse)
        out = torch.cat(outs, dim=0) if len(outs) > 1 else outs[0]
        ctx.save_for_backward(q, k, v, out, *lses)
        ctx.meta = (scale, zigzag, S, nq, nkv, hd)
        return out.view(1, S, nq, hd)

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, *lses = ctx.saved_tensors
        scale, zigzag, S, nq, nkv, hd = ctx.meta
        W = nkv * hd
        ex = CPExchange.get(S, W)
        St = S * ex.world
        full = ex.gather(k.view(S, W), v.view(S, W), zigzag)
        kf, vf = full[0].view(1, St, nkv, hd), full[1].view(1, St, nkv, hd)
        dout = dout.contiguous().view(S, nq * hd)
        dfull = ex.dfull
        dq = torch.empty_like(q)
        segs = _segments(ex.rank, ex.world, S, zigzag)
        tmp = None
        for i, (a, b, off) in enumerate(segs):
            kend = off + (b - a)
            if i == 0:
                dst = dfull
                if kend < St:
                    dfull[:, kend:].zero_()
            else:
                tmp = torch.empty(2, kend, W, dtype=torch.bfloat16, device=q.device) if tmp is None else tmp
                dst = tmp
            dk = dst[0, :kend].view(1, kend, nkv, hd)
            dv = dst[1, :kend].view(1, kend, nkv, hd)
            dq[:, a:b] = A.rect_backward(q[:, a:b], kf[:, :kend], vf[:, :kend], out[a:b], lses[i], dout[a:b], dk, dv,
                                         off, True, scale)
            if i > 0:
                dfull[:, :kend] += tmp[:, :kend]
        red = ex.reduce_scatter(zigzag)
        return dq, red[0].view(1, S, nkv, hd), red[1].view(1, S, nkv, hd), None, None


def supported(q, k, v) -> bool:
    cp = ps.get_context_parallel_world_size()
    return (q.is_cuda and q.shape[0] == 1 and A.rect_supported(q, k, v) and cp <= 16
            and (q.shape[1] // 2) % 128 == 0 and k.shape[2] * k.shape[3] % 8 == 0)


def fused_cp_attention(q, k, v, scale, zigzag: bool = False):
    """q ``[1, S_local, nq, 128]``, k/v ``[1, S_local, nkv, 128]`` → ``[1, S_local, nq, 128]`` (causal over the whole
    sequence; with ``zigzag`` the local tokens are chunks ``r`` and ``2·cp−1−r`` of ``2·cp``)."""
    return _FusedCPAttention.apply(q, k, v, float(scale), bool(zigzag))


def zigzag_slice(x: torch.Tensor, cp: int, rank: int, dim: int = 1) -> torch.Tensor:
    """This rank's tokens of a full-sequence tensor under the zig-zag layout (use it on ids, labels, positions)."""
    chunks = x.chunk(2 * cp, dim=dim)
    return torch.cat([chunks[rank], chunks[2 * cp - 1 - rank]], dim=dim)
