"""MoE dispatch / combine on the device-side exchange kernels of ``ops/csrc/moe_ep.cu``.

Forward of one layer:  rank → plan (count exchange) → scatter (permute + send by peer stores) → barrier →
grouped expert GEMMs → barrier → gather (receive by peer loads + weighted unpermute). The backward runs the same
kernels with the roles swapped (the gradient of a gather is a weighted scatter and vice versa). No split size ever
reaches the host, so a layer costs no device→host copy and no host synchronisation — the all-to-all-v path of the
reference needs one per layer (``training_graph/transformer/moe/token_dispatcher.py:130-159``).

With a single expert-parallel rank the kernels are the local permute / unpermute and touch no flags; row buffers
are then ordinary tensors. With ``ep > 1`` each MoE layer owns two row buffers in peer-mapped memory (expert input
and expert output, both needed again by the backward pass) and the group shares two more for gradients.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..ops import _lib
from . import parallel_state as ps
from ..tools.logger import logger
from . import symm_mem
from ..ops.functional import apply_fn

BLOCK = 128


class _Plan:
    """What ``GroupedMLP`` needs from a permutation plan (all device tensors)."""

    def __init__(self, E_local, rows_cap, dev):
        self.group_offsets = torch.zeros(E_local + 1, dtype=torch.int32, device=dev)
        self.seg_fill = torch.zeros(E_local, dtype=torch.int32, device=dev)
        self.block_group = torch.zeros(rows_cap // BLOCK, dtype=torch.int32, device=dev)
        self.num_blocks = torch.zeros(1, dtype=torch.int32, device=dev)
        self.rows = rows_cap


STATUS_MOE_OVERFLOW = 6      # kStatusMoeOverflow of ops/csrc/moe_ep.cu


def adapt_capacity() -> bool:
    """``MoEExchange.adapt_capacity`` of every live exchange (see there)."""
    grew = False
    for ex in list(MoEExchange._instances.values()):
        grew = ex.adapt_capacity() or grew
    return grew


class MoEExchange:
    """Per-group state: flags, count table, shared gradient row buffers, epoch counter."""

    _instances: Dict[tuple, "MoEExchange"] = {}

    @classmethod
    def get(cls, config) -> "MoEExchange":
        grp = ps.get_expert_model_parallel_group()
        key = (id(grp), config.hidden_size, config.num_moe_experts, config.moe_router_topk)
        inst = cls._instances.get(key)
        if inst is None:
            inst = cls._instances[key] = cls(config, grp)
        return inst

    def __init__(self, config, group):
        self.group = group
        self.world = ps.get_expert_model_parallel_world_size()
        self.rank = ps.get_expert_model_parallel_rank()
        self.E = config.num_moe_experts
        self.E_local = self.E // self.world
        self.k = config.moe_router_topk
        self.H = config.hidden_size
        self.factor = float(getattr(config, "moe_ep_buffer_factor", 1.25) or 1.25)
        self.dev = torch.device("cuda", torch.cuda.current_device())
        # epoch of the flag protocol: a device counter that the plan / barrier kernels advance themselves, so the
        # same launches can be replayed from a CUDA graph
        self.epoch_ctr = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.lib = _lib.get_lib()
        self._arr = ctypes.c_longlong * self.world
        self._shared: Dict[tuple, object] = {}
        self._in_flight: Dict[object, set] = {}
        self._symm_names: list = []
        self.alloc_rows = None      # rows of the symmetric row buffers, agreed over the group
        if self.world > 1:
            words = self.lib.mfb_moe_flag_words()
            flags = symm_mem.allocate(f"moe.flags.{id(group)}.{self.H}.{self.E}.{self.k}", words * 4, group, self.dev)
            flags.tensor.zero_()
            table = symm_mem.allocate(f"moe.table.{id(group)}.{self.H}.{self.E}.{self.k}", self.world * (self.E + 1) * 4, group, self.dev)
            table.tensor.zero_()
            self.flags, self.table = flags, table
            self.peer_flags = self._arr(*[int(p) for p in flags.ptrs])
            self.peer_table = self._arr(*[int(p) for p in table.ptrs])
            torch.cuda.synchronize()
            dist.barrier(group=group)
        else:
            self.peer_flags = self.peer_table = None

    # ------------------------------------------------------------------------------------------------
    def rows_cap(self, T: int) -> int:
        """Rows of this rank's receive buffers for ``T`` local tokens.

        Symmetric allocations must have one size on all ranks, so the first call, the first one after a growth and
        every call that asks for more rows than were agreed so far settle the size with one all-reduce and a host
        read. Routing that still overflows the buffers is repaired by ``adapt_capacity``."""
        factor = self.factor
        if not torch.is_grad_enabled():
            # inference has no step boundary at which to grow the buffers and holds one pair of them for all layers,
            # so it starts from a roomier bound
            # so it takes the worst case (every token of the group routed to this rank: nothing can be dropped)
            # while that stays within a few GB, and a roomier bound otherwise; ``generate`` checks the overflow
            # flag at its final synchronisation and raises if rows were dropped
            worst = float(self.world)
            factor = worst if T * self.k * worst * self.H * 2 <= (8 << 30) else max(factor, min(worst, 2.5))
        cap = int(T * self.k * (factor if self.world > 1 else 1.0)) + self.E_local * (BLOCK - 1)
        cap = (cap + BLOCK - 1) // BLOCK * BLOCK
        if self.world <= 1:
            return cap
        if self.alloc_rows is None or cap > self.alloc_rows:
            # a larger token count than ever before (first call, or a longer prefill): all ranks reach this point in
            # the same call because the token count per rank is the same over the group
            t = torch.tensor([cap], dtype=torch.int64, device=self.dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
            self.alloc_rows = int(t.item())
        return min(cap, self.alloc_rows)

    def row_buffer(self, tag: str, rows: int):
        """``(tensor [rows, H] bf16, peer pointer array)``; peer-mapped when the group has more than one rank (then
        the allocation has ``alloc_rows`` rows on every rank and the first ``rows`` are returned)."""
        hit = self._shared.get(tag)
        if hit is not None and hit[0].shape[0] >= rows:
            return hit[0][:rows], hit[1]
        if self.world > 1:
            full = max(self.alloc_rows or rows, rows)
            name = f"moe.{tag}.{full}.{self.H}.{self.E}.{id(self.group)}"
            self._symm_names.append(name)
            buf = symm_mem.allocate(name, full * self.H * 2, self.group, self.dev)
            t = buf.tensor.view(torch.bfloat16)[:full * self.H].view(full, self.H)
            ptrs = self._arr(*[int(p) for p in buf.ptrs])
        else:
            t = torch.empty(rows, self.H, dtype=torch.bfloat16, device=self.dev)
            ptrs = self._arr(t.data_ptr())
        self._shared[tag] = (t, ptrs)
        return t[:rows], ptrs

    def acquire_slot(self, layer_key) -> int:
        """Row buffers of a layer stay in use from its forward to the end of its backward; a second forward of
        the same layer before that (pipeline schedules, recompute) gets the next free slot."""
        used = self._in_flight.setdefault(layer_key, set())
        slot = 0
        while slot in used:
            slot += 1
        used.add(slot)
        return slot

    def release_slot(self, layer_key, slot: int):
        self._in_flight.get(layer_key, set()).discard(slot)

    def local_ptrs(self, t: torch.Tensor):
        return self._arr(t.data_ptr())

    def status(self):
        return _lib.status_word(self.dev).data_ptr()

    def adapt_capacity(self) -> bool:
        """Grow the receive buffers if a rank got more rows than they hold (the plan kernel then set the overflow
        code in the status word and the scatter skipped the rows that did not fit).

        Collective over the expert-parallel group and synchronising: call it between steps. All ranks grow together
        because the row buffers are symmetric allocations. Returns True if the factor changed; the dropped rows of
        the step that overflowed are not recomputed.
        """
        if self.world <= 1:
            return False
        word = _lib.status_word(self.dev)
        flag = word[1:2].clone()
        dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.group)
        if int(flag.item()) == 0:
            return False
        word[1:2].zero_()
        old = self.factor
        self.factor = min(self.factor * 1.5, float(self.world))
        if self.factor == old:
            logger.warning("expert-parallel receive buffers overflow at the maximum factor %.2f", old)
            return False
        for name in self._symm_names:
            symm_mem.free(name, self.group)
        self._symm_names.clear()
        self._shared.clear()
        self.alloc_rows = None
        logger.warning("expert-parallel receive buffers overflowed: moe_ep_buffer_factor %.2f -> %.2f "
                       "(set it in the model config to avoid the dropped rows of the first steps)", old, self.factor)
        return True

    # ---- kernel wrappers ------------------------------------------------------------------------------
    def plan(self, ids: torch.Tensor, T: int):
        n = ids.numel()
        rows = self.rows_cap(T)
        st = _PlanState(self, rows, n)
        rc = self.lib.mfb_moe_rank(ids.data_ptr(), n, self.E, st.rank_in_e.data_ptr(), st.counts.data_ptr(), _lib.stream_ptr())
        _lib.check(rc, "mfb_moe_rank")
        rc = self.lib.mfb_moe_plan(self.world, self.rank, self.epoch_ctr.data_ptr(), self.E, self.E_local, rows, st.counts.data_ptr(),
                                   self.peer_table, self.peer_flags, st.write_base.data_ptr(), st.owner_cap.data_ptr(),
                                   st.plan.group_offsets.data_ptr(), st.plan.seg_fill.data_ptr(),
                                   st.plan.block_group.data_ptr(), st.plan.num_blocks.data_ptr(), self.status(),
                                   _lib.stream_ptr())
        _lib.check(rc, "mfb_moe_plan")
        _lib.count_launch(2)
        return st

    def scatter(self, st, x, ids, peer_ptrs, weights=None, zero_pad: bool = True):
        """``zero_pad=False`` (forward-only calls) leaves the padding rows of the expert segments as they are: rows
        are independent in every expert operator and padding rows are never gathered; only the weight-gradient
        GEMM, which sums over rows, needs them to be zero."""
        T = x.shape[0]
        rc = self.lib.mfb_moe_scatter(self.world, self.rank, T, self.k, self.H, self.E_local, st.rows, x.data_ptr(),
                                      ids.data_ptr(), st.rank_in_e.data_ptr(), st.write_base.data_ptr(),
                                      st.owner_cap.data_ptr(), peer_ptrs,
                                      _lib.ptr(weights), st.dest_row.data_ptr(),
                                      st.plan.group_offsets.data_ptr() if zero_pad else 0,
                                      st.plan.seg_fill.data_ptr() if zero_pad else 0, self.status(), _lib.stream_ptr())
        _lib.check(rc, "mfb_moe_scatter")
        _lib.count_launch()

    def barrier(self, phase: int):
        if self.world > 1:
            rc = self.lib.mfb_moe_barrier(self.world, self.rank, self.epoch_ctr.data_ptr(), phase, self.peer_flags, self.status(),
                                          _lib.stream_ptr())
            _lib.check(rc, "mfb_moe_barrier")
            _lib.count_launch()

    def gather(self, st, T, ids, peer_ptrs, weights=None, g=None):
        out = torch.empty(T, self.H, dtype=torch.bfloat16, device=self.dev)
        dots = torch.empty(T, self.k, dtype=torch.float32, device=self.dev) if g is not None else None
        rc = self.lib.mfb_moe_gather(self.world, self.rank, T, self.k, self.H, self.E_local, st.rows, out.data_ptr(),
                                     ids.data_ptr(), st.dest_row.data_ptr(), peer_ptrs, _lib.ptr(weights), _lib.ptr(g),
                                     _lib.ptr(dots), self.status(), _lib.stream_ptr())
        _lib.check(rc, "mfb_moe_gather")
        _lib.count_launch()
        return out, dots


class _PlanState:
    def __init__(self, ex: MoEExchange, rows: int, n: int):
        dev = ex.dev
        self.rows = rows
        self.rank_in_e = torch.empty(n, dtype=torch.int32, device=dev)
        self.counts = torch.empty(ex.E, dtype=torch.int32, device=dev)
        self.write_base = torch.empty(ex.E, dtype=torch.int32, device=dev)
        self.owner_cap = torch.zeros(8, dtype=torch.int32, device=dev)
        self.dest_row = torch.empty(n, dtype=torch.int32, device=dev)
        self.plan = _Plan(ex.E_local, rows, dev)


class _Dispatch(torch.autograd.Function):
    """``x [T,H]`` → expert input rows of this rank ``[rows, H]`` (permute + send)."""

    @staticmethod
    def forward(ctx, x, ids, ex: MoEExchange, st: _PlanState, layer_key):
        x = x.contiguous()
        T = x.shape[0]
        if ex.world > 1:
            xin, ptrs = ex.row_buffer(f"xin.{layer_key}", st.rows)
        else:
            xin = torch.empty(st.rows, ex.H, dtype=torch.bfloat16, device=x.device)
            ptrs = ex.local_ptrs(xin)
        ex.scatter(st, x, ids, ptrs, zero_pad=not str(layer_key).startswith("nograd"))
        ex.barrier(1)
        ctx.ex, ctx.st, ctx.T = ex, st, T
        ctx.save_for_backward(ids)
        return xin

    @staticmethod
    def backward(ctx, dxin):
        ex, st, T = ctx.ex, ctx.st, ctx.T
        (ids,) = ctx.saved_tensors
        dxin = dxin.contiguous()
        if ex.world > 1:
            ws, ptrs = ex.row_buffer("dx_ws", st.rows)
            ws.copy_(dxin)
            ex.barrier(2)
        else:
            ptrs = ex.local_ptrs(dxin)
        dx, _ = ex.gather(st, T, ids, ptrs)
        ex.release_slot(*st.slot)
        return dx, None, None, None, None


class _Combine(torch.autograd.Function):
    """Expert output rows ``[rows, H]`` + ``probs [T,k]`` → ``[T,H]`` (receive + weighted unpermute)."""

    @staticmethod
    def forward(ctx, y, probs, ids, ex: MoEExchange, st: _PlanState, layer_key):
        T = probs.shape[0]
        probs = probs.contiguous().float()
        if ex.world > 1:
            yout, ptrs = ex.row_buffer(f"yout.{layer_key}", st.rows)
            yout.copy_(y)
            ex.barrier(2)
        else:
            yout, ptrs = y.contiguous(), None
            ptrs = ex.local_ptrs(yout)
        out, _ = ex.gather(st, T, ids, ptrs, weights=probs)
        ctx.ex, ctx.st, ctx.T, ctx.ptrs = ex, st, T, ptrs
        ctx.save_for_backward(ids, probs, yout)
        return out

    @staticmethod
    def backward(ctx, dout):
        ex, st, T = ctx.ex, ctx.st, ctx.T
        ids, probs, yout = ctx.saved_tensors
        dout = dout.contiguous()
        # d(probs)[t,j] = <dout[t], y_row(t,j)>: rows are still in the owners' output buffers
        _, dots = ex.gather(st, T, ids, ctx.ptrs, weights=None, g=dout)
        if ex.world > 1:
            dy, ptrs = ex.row_buffer("dy_ws", st.rows)
        else:
            dy = torch.empty(st.rows, ex.H, dtype=torch.bfloat16, device=dout.device)
            ptrs = ex.local_ptrs(dy)
        ex.scatter(st, dout, ids, ptrs, weights=probs)
        ex.barrier(1)
        # peers overwrite dy_ws only after this rank has passed the barrier of this layer's dispatch backward,
        # which comes after the expert GEMMs that consume it
        return dy, dots, None, None, None, None


def supported(config, hidden: torch.Tensor) -> bool:
    return (hidden.is_cuda and hidden.dtype == torch.bfloat16 and hidden.dim() == 2 and hidden.shape[1] % 8 == 0
            and config.num_moe_experts <= 512 and ps.get_expert_model_parallel_world_size() <= 8)


def moe_dispatch_experts_combine(layer, hidden: torch.Tensor, probs: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """Router outputs → combined expert outputs ``[T, H]`` through the fused exchange."""
    ex = MoEExchange.get(layer.config)
    ids = ids.contiguous()
    st = ex.plan(ids, hidden.shape[0])
    needs_grad = torch.is_grad_enabled() and (hidden.requires_grad or probs.requires_grad)
    # forward-only calls share one pair of row buffers between all layers: a layer's combine barrier orders every
    # peer's reads before the next layer's writes. With gradients the buffers live until the layer's backward.
    layer_key = layer.layer_number if needs_grad else "nograd"
    slot = ex.acquire_slot(layer_key)
    st.slot = (layer_key, slot)
    key = f"{layer_key}.{slot}"
    xin = apply_fn(_Dispatch, hidden, ids, ex, st, key)
    layer.last_tokens_per_expert = st.counts
    y = layer.experts(xin, st.plan)
    out = apply_fn(_Combine, y, probs, ids, ex, st, key)
    if not needs_grad:
        ex.release_slot(*st.slot)
    return out
