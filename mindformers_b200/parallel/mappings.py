"""Differentiable collectives between tensor-parallel / sequence-parallel regions.

Explicit counterparts of what the reference obtains from the MindSpore auto-parallel compiler in
training (shard strategies at ``training_graph/tensor_parallel/layers.py:248-263,402-419``) and writes
by hand in inference (``inference/tensor_parallel/mappings.py:21-92``). Activations are ``[T, H]``
(tokens first); sequence parallelism shards the token axis.

These NCCL versions are the baseline data plane. The fused compute+collective kernels in
``parallel/fused_comm.py`` replace the (all-gather, GEMM) and (GEMM, reduce-scatter) pairs.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import parallel_state as ps
from ..ops.functional import apply_fn


def _tp():
    return ps.get_tensor_model_parallel_group(), ps.get_tensor_model_parallel_world_size()


def all_gather_first_dim(x: torch.Tensor, group, world: int) -> torch.Tensor:
    if world == 1:
        return x
    x = x.contiguous()
    out = torch.empty((x.shape[0] * world, *x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x, group=group)
    return out


def reduce_scatter_first_dim(x: torch.Tensor, group, world: int) -> torch.Tensor:
    if world == 1:
        return x
    x = x.contiguous()
    if x.shape[0] % world != 0:
        raise ValueError(f"first dimension {x.shape[0]} is not divisible by the group size {world}")
    out = torch.empty((x.shape[0] // world, *x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.reduce_scatter_tensor(out, x, group=group)
    return out


def all_reduce(x: torch.Tensor, group, world: int) -> torch.Tensor:
    if world == 1:
        return x
    x = x.contiguous()
    dist.all_reduce(x, group=group)
    return x


class _CopyToTP(torch.autograd.Function):
    """Identity forward, all-reduce backward (input of a column-parallel layer without SP)."""
    @staticmethod
    def forward(ctx, x):
        return x

    @staticmethod
    def backward(ctx, g):
        grp, n = _tp()
        return all_reduce(g.clone() if n > 1 else g, grp, n)


class _ReduceFromTP(torch.autograd.Function):
    """All-reduce forward, identity backward (output of a row-parallel layer without SP)."""
    @staticmethod
    def forward(ctx, x):
        grp, n = _tp()
        return all_reduce(x, grp, n)

    @staticmethod
    def backward(ctx, g):
        return g


class _GatherFromSP(torch.autograd.Function):
    """All-gather tokens forward, reduce-scatter (or split) backward."""
    @staticmethod
    def forward(ctx, x, reduce_scatter_grad):
        ctx.rs = reduce_scatter_grad
        grp, n = _tp()
        return all_gather_first_dim(x, grp, n)

    @staticmethod
    def backward(ctx, g):
        grp, n = _tp()
        if ctx.rs:
            return reduce_scatter_first_dim(g, grp, n), None
        r = ps.get_tensor_model_parallel_rank()
        chunk = g.shape[0] // n
        return g[r * chunk:(r + 1) * chunk].contiguous(), None


class _ReduceScatterToSP(torch.autograd.Function):
    """Reduce-scatter tokens forward, all-gather backward."""
    @staticmethod
    def forward(ctx, x):
        grp, n = _tp()
        return reduce_scatter_first_dim(x, grp, n)

    @staticmethod
    def backward(ctx, g):
        grp, n = _tp()
        return all_gather_first_dim(g, grp, n)


class _ScatterToSP(torch.autograd.Function):
    """Keep this rank's token chunk forward, all-gather backward."""
    @staticmethod
    def forward(ctx, x):
        n = ps.get_tensor_model_parallel_world_size()
        if n == 1:
            return x
        r = ps.get_tensor_model_parallel_rank()
        chunk = x.shape[0] // n
        return x[r * chunk:(r + 1) * chunk].contiguous()

    @staticmethod
    def backward(ctx, g):
        grp, n = _tp()
        return all_gather_first_dim(g, grp, n)


class _GatherLastDim(torch.autograd.Function):
    """All-gather the feature axis forward (column-parallel ``gather_output``), split backward."""
    @staticmethod
    def forward(ctx, x):
        grp, n = _tp()
        if n == 1:
            return x
        parts = [torch.empty_like(x) for _ in range(n)]
        dist.all_gather(parts, x.contiguous(), group=grp)
        return torch.cat(parts, dim=-1)

    @staticmethod
    def backward(ctx, g):
        n = ps.get_tensor_model_parallel_world_size()
        if n == 1:
            return g
        r = ps.get_tensor_model_parallel_rank()
        return g.chunk(n, dim=-1)[r].contiguous()


class _AllToAll(torch.autograd.Function):
    """All-to-all with explicit split sizes over an arbitrary group; backward swaps the splits."""
    @staticmethod
    def forward(ctx, x, out_splits, in_splits, group):
        ctx.group, ctx.out_splits, ctx.in_splits = group, out_splits, in_splits
        world = dist.get_world_size(group) if group is not None else 1
        if world == 1:
            return x
        x = x.contiguous()
        n_out = sum(out_splits) if out_splits is not None else x.shape[0]
        out = torch.empty((n_out, *x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_to_all_single(out, x, output_split_sizes=out_splits, input_split_sizes=in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        return _AllToAll.apply(g, ctx.in_splits, ctx.out_splits, ctx.group), None, None, None


def copy_to_tensor_model_parallel_region(x): return apply_fn(_CopyToTP, x)
def reduce_from_tensor_model_parallel_region(x): return apply_fn(_ReduceFromTP, x)
def gather_from_sequence_parallel_region(x, reduce_scatter_grad=True): return apply_fn(_GatherFromSP, x, reduce_scatter_grad)
def reduce_scatter_to_sequence_parallel_region(x): return apply_fn(_ReduceScatterToSP, x)
def scatter_to_sequence_parallel_region(x): return apply_fn(_ScatterToSP, x)
def gather_from_tensor_model_parallel_region(x): return apply_fn(_GatherLastDim, x)
def all_to_all(x, out_splits, in_splits, group): return _AllToAll.apply(x, out_splits, in_splits, group)
