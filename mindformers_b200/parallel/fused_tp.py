"""Tensor-parallel linear layers whose collective runs inside the GEMM kernel (``ops/csrc/fused_tp_gemm.cu``).

``allgather_linear``: ``y[T, N/tp] = all_gather(x[T/tp, K]) @ W^T`` — the sequence-parallel input of a
column-parallel layer. ``linear_reduce_scatter``: ``y[T/tp, N] = reduce_scatter(x[T, K/tp] @ W^T)`` — the
output of a row-parallel layer. The backward pass of each one is the other kernel (dgrad) plus a plain
weight-gradient GEMM on the gathered operand that the forward (or the backward gather) left in local memory.

Peer-mapped buffers come from ``symm_mem``; flags carry a per-kernel call counter ("epoch") that every rank
advances identically.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..ops import _lib
from ..ops import functional as Fn
from . import parallel_state as ps
from . import symm_mem

_lib.optional_entry("mfb_tp_allgather_gemm",
                    [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                     ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                     ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                     ctypes.c_void_p, ctypes.c_void_p])
_lib.optional_entry("mfb_tp_gemm_reduce_scatter",
                    [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                     ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                     ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                     ctypes.c_void_p, ctypes.c_void_p])


_lib.optional_entry("mfb_tp_allreduce_ksplit", [ctypes.c_int, ctypes.c_int, ctypes.c_int])
_lib.optional_entry("mfb_tp_gemm_allreduce",
                    [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                     ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                     ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                     ctypes.c_void_p, ctypes.c_void_p])

AR_FLAG_TILES = 8192          # tiles per call that the all-reduce flag arrays have room for
AR_MAX_ROWS = 4096            # above this the two-step path (reduce-scatter + all-gather) moves fewer bytes


class TpCommContext:
    """Symmetric buffers and epochs of one tensor-parallel group."""

    def __init__(self, group, tp: int, rank: int, device):
        self.group, self.tp, self.rank, self.device = group, tp, rank, device
        self.ag_epoch = 0
        self.rs_epoch = 0
        self.x_elems = 0
        self.recv_elems = 0
        self.flags = None
        self.xs = None
        self.recv = None
        self.max_tiles = 0
        self.ar_epoch = 0
        self.ar_flags = None
        self.ar_recv = None
        self.ar_elems = 0
        self.ar_arrays = None

    def _ptr_array(self, ptrs):
        arr = (ctypes.c_void_p * 8)()
        for i, p in enumerate(ptrs):
            arr[i] = int(p)
        return arr

    def ensure(self, x_elems: int, recv_elems: int, tiles: int):
        """(Re)allocate buffers when a larger problem shows up; collective over the TP group."""
        if self.flags is None or tiles > self.max_tiles:
            self.max_tiles = max(tiles, 4096)
            n_ints = self.tp + 2 * self.tp * self.max_tiles
            self.flags = symm_mem.allocate(f"tp_flags_{self.max_tiles}", n_ints * 4, self.group, self.device)
            self.flags.tensor.zero_()
            torch.cuda.synchronize()
            self.flags.handle.barrier()
            self.ag_epoch = self.rs_epoch = 0
        if x_elems > self.x_elems:
            self.x_elems = x_elems
            self.xs = symm_mem.allocate(f"tp_xs_{x_elems}", 2 * x_elems * 2, self.group, self.device)
        if recv_elems > self.recv_elems:
            self.recv_elems = recv_elems
            self.recv = symm_mem.allocate(f"tp_recv_{recv_elems}", 2 * self.tp * recv_elems * 2, self.group, self.device)
            torch.cuda.synchronize()
            self.recv.handle.barrier()

    def ensure_allreduce(self, elems: int):
        """Receive slots (2 parities x tp ranks x ``elems`` bf16) and tile flags of the one-shot all-reduce;
        collective over the TP group when something has to be allocated."""
        if self.ar_flags is None:
            self.ar_flags = symm_mem.allocate("tp_ar_flags", 2 * self.tp * 8 * AR_FLAG_TILES * 4, self.group, self.device)
            self.ar_flags.tensor.zero_()
            torch.cuda.synchronize()
            self.ar_flags.handle.barrier()
        if elems > self.ar_elems:
            self.ar_elems = elems
            self.ar_recv = symm_mem.allocate(f"tp_ar_recv_{elems}", 2 * self.tp * elems * 2, self.group, self.device)
            torch.cuda.synchronize()
            self.ar_recv.handle.barrier()

    # views into the flag buffer (ints)
    def ready_ptrs(self):
        return [p for p in self.flags.ptrs]

    def tile_flag_ptrs(self):
        return [p + self.tp * 4 for p in self.flags.ptrs]


_CTX: Optional[TpCommContext] = None


def context() -> TpCommContext:
    global _CTX
    if _CTX is None:
        grp = ps.get_tensor_model_parallel_group()
        _CTX = TpCommContext(grp, ps.get_tensor_model_parallel_world_size(), ps.get_tensor_model_parallel_rank(),
                             torch.device("cuda", torch.cuda.current_device()))
        symm_mem.enable()
    return _CTX


def _n_blocks(N: int) -> int:
    return (N + 255) // 256 if N >= 256 else (N + 127) // 128


def allgather_gemm(x_local: torch.Tensor, w: torch.Tensor, b_mn: bool = False):
    """Returns ``(y [T, N], x_full [T, K])``; ``w`` is ``[N, K]`` (or ``[K, N]`` with ``b_mn``)."""
    ctx = context()
    tp, rank = ctx.tp, ctx.rank
    Tl, K = x_local.shape
    T = Tl * tp
    N = w.shape[1] if b_mn else w.shape[0]
    ctx.ensure(Tl * K, 0, 0)
    ctx.ag_epoch += 1
    e = ctx.ag_epoch
    slot = e & 1
    xs_local = ctx.xs.tensor.view(torch.bfloat16)[slot * ctx.x_elems: slot * ctx.x_elems + Tl * K].view(Tl, K)
    xs_local.copy_(x_local)
    peer = [p + slot * ctx.x_elems * 2 for p in ctx.xs.ptrs]
    x_full = torch.empty((T, K), dtype=torch.bfloat16, device=x_local.device)
    y = torch.empty((T, N), dtype=torch.bfloat16, device=x_local.device)
    block_flags = torch.empty(T // 128, dtype=torch.int32, device=x_local.device)
    ready = ctx.ready_ptrs()
    st = _lib.status_word(x_local.device)
    rc = _lib.get_lib().mfb_tp_allgather_gemm(ctx._ptr_array(peer), K, x_full.data_ptr(), w.data_ptr(), y.data_ptr(),
                                              T, N, K, w.stride(0), y.stride(0), int(b_mn), tp, rank, e,
                                              block_flags.data_ptr(), ready[rank], ctx._ptr_array(ready),
                                              st.data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "mfb_tp_allgather_gemm")
    _lib.count_launch()
    return y, x_full


def gemm_reduce_scatter(x: torch.Tensor, w: torch.Tensor, b_mn: bool = False) -> torch.Tensor:
    """``reduce_scatter_rows(x @ W^T)``: ``x`` ``[T, K_local]``, ``w`` ``[N, K_local]`` (or ``[K_local, N]``)."""
    ctx = context()
    tp, rank = ctx.tp, ctx.rank
    T, K = x.shape
    N = w.shape[1] if b_mn else w.shape[0]
    Tl = T // tp
    tiles = (Tl // 128) * _n_blocks(N)
    ctx.ensure(0, Tl * N, tiles)
    ctx.rs_epoch += 1
    e = ctx.rs_epoch
    if not x.is_contiguous():
        x = x.contiguous()
    y = torch.empty((Tl, N), dtype=torch.bfloat16, device=x.device)
    recv = list(ctx.recv.ptrs)
    tf = ctx.tile_flag_ptrs()
    # the receive slots of this call are laid out with the actual slot size
    st = _lib.status_word(x.device)
    rc = _lib.get_lib().mfb_tp_gemm_reduce_scatter(x.data_ptr(), w.data_ptr(), y.data_ptr(), T, N, K, x.stride(0),
                                                   w.stride(0), y.stride(0), int(b_mn), tp, rank, e, recv[rank],
                                                   ctx._ptr_array(recv), tf[rank], ctx._ptr_array(tf), st.data_ptr(),
                                                   _lib.stream_ptr())
    _lib.check(rc, "mfb_tp_gemm_reduce_scatter")
    _lib.count_launch()
    return y


def gemm_all_reduce(x: torch.Tensor, w: torch.Tensor, b_mn: bool = False) -> torch.Tensor:
    """``all_reduce(x @ W^T)`` with identical bits on every rank: ``x`` ``[T, K_local]`` (any ``T``), ``w``
    ``[N, K_local]`` (or ``[K_local, N]``). The row-parallel layers of tensor-parallel inference use it
    (reference: ``parallel_core/inference/tensor_parallel/layers.py`` ``RowParallelLinear`` + all-reduce)."""
    ctx = context()
    tp, rank = ctx.tp, ctx.rank
    T, K = x.shape
    N = w.shape[1] if b_mn else w.shape[0]
    rows = (T + 127) // 128 * 128
    ksplit = _lib.get_lib().mfb_tp_allreduce_ksplit(T, N, K)     # decode: several CTAs share the K range of a tile
    ctx.ensure_allreduce(ksplit * rows * N)
    ctx.ar_epoch += 1
    if not x.is_contiguous():
        x = x.contiguous()
    y = torch.empty((T, N), dtype=torch.bfloat16, device=x.device)
    cached = ctx.ar_arrays
    if cached is None or cached[0] is not ctx.ar_recv:
        recv, tf = list(ctx.ar_recv.ptrs), list(ctx.ar_flags.ptrs)
        cached = ctx.ar_arrays = (ctx.ar_recv, recv[rank], ctx._ptr_array(recv), tf[rank], ctx._ptr_array(tf))
    _, recv_local, recv_arr, tf_local, tf_arr = cached
    st = _lib.status_word(x.device)
    rc = _lib.get_lib().mfb_tp_gemm_allreduce(x.data_ptr(), w.data_ptr(), y.data_ptr(), T, N, K, x.stride(0),
                                              w.stride(0), y.stride(0), int(b_mn), tp, rank, ctx.ar_epoch, recv_local,
                                              recv_arr, tf_local, tf_arr, AR_FLAG_TILES,
                                              st.data_ptr(), _lib.stream_ptr())
    _lib.check(rc, "mfb_tp_gemm_allreduce")
    _lib.count_launch()
    return y


def allreduce_shapes_ok(T: int, K: int, N: int) -> bool:
    tiles = ((T + 127) // 128) * ((N + 127) // 128)
    return 1 <= T <= AR_MAX_ROWS and K % 8 == 0 and N >= 128 and N % 64 == 0 and tiles <= AR_FLAG_TILES


class _AllGatherLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_local, w):
        from .recompute import cached_output
        y, x_full = cached_output(lambda: allgather_gemm(x_local, w))    # no second exchange in a recomputation
        ctx.save_for_backward(x_full, w)
        return y

    @staticmethod
    def backward(ctx, dy):
        x_full, w = ctx.saved_tensors
        dy = dy.contiguous()
        # dgrad: partial dx over ranks, reduce-scattered along tokens inside the GEMM
        dx = gemm_reduce_scatter(dy, w, b_mn=True)
        main_grad = getattr(w, "main_grad", None)
        if main_grad is not None:
            Fn.gemm(dy, x_full, a_mn=True, b_mn=True, out=main_grad, accumulate=True)
            dw = None
        else:
            dw = Fn.gemm(dy, x_full, a_mn=True, b_mn=True, out_dtype=w.dtype)
        return dx, dw


class _LinearReduceScatterFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        from .recompute import cached_output
        ctx.save_for_backward(x, w)
        return cached_output(lambda: gemm_reduce_scatter(x, w))

    @staticmethod
    def backward(ctx, dy_local):
        x, w = ctx.saved_tensors
        dx, dy_full = allgather_gemm(dy_local.contiguous(), w, b_mn=True)
        main_grad = getattr(w, "main_grad", None)
        if main_grad is not None:
            Fn.gemm(dy_full, x, a_mn=True, b_mn=True, out=main_grad, accumulate=True)
            dw = None
        else:
            dw = Fn.gemm(dy_full, x, a_mn=True, b_mn=True, out_dtype=w.dtype)
        return dx, dw


def shapes_ok(T_total: int, K: int, N: int, tp: int) -> bool:
    return T_total % (tp * 128) == 0 and K % 8 == 0 and N >= 128 and N % 64 == 0


def allgather_linear(x_local: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return _AllGatherLinearFn.apply(x_local, w)


def linear_reduce_scatter(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return _LinearReduceScatterFn.apply(x, w)
