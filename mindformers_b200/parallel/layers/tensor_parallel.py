"""Tensor-parallel linear layers and the vocab-parallel embedding.

API of the reference's ``training_graph/tensor_parallel/layers.py`` (``VocabParallelEmbedding`` :39,
``ColumnParallelLinear`` :106, ``RowParallelLinear`` :283, ``LinearNoTP`` :439) and of
``inference/tensor_parallel/layers.py`` (:44-659), one implementation for training and inference.
Weights are ``[out, in]``; ``forward`` returns ``(output, bias)`` with the bias returned instead of
added when ``skip_bias_add`` is set. Under sequence parallelism the column layer all-gathers tokens
before its GEMM and the row layer reduce-scatters after it; with ``config.fused_tp_comm`` those pairs
run as one kernel over NVLink peer memory (see ``parallel/fused_comm.py``).
"""
from __future__ import annotations

import math
from typing import Callable, Optional

import torch
import torch.nn as nn

from ...ops import functional as Fn
from .. import mappings as M
from .. import parallel_state as ps


def section_local_sizes(sections, world: int, groups=None):
    """Rows of each section that one rank holds. ``groups[i]`` is the number of indivisible groups (heads) of
    section ``i``; a section with fewer groups than ranks is replicated: each rank holds one whole group."""
    out = []
    for i, size in enumerate(sections):
        g = groups[i] if groups else None
        if g and g < world:
            if world % g or size % g:
                raise ValueError(f"section of {g} groups cannot be replicated over {world} ranks")
            out.append(size // g)
        else:
            if size % world:
                raise ValueError(f"section of size {size} is not divisible by {world}")
            out.append(size // world)
    return out


def shard_sections(w: torch.Tensor, sections, dim: int, rank: int, world: int, groups=None) -> torch.Tensor:
    """Split ``w`` along ``dim`` into ``sections`` (e.g. q|k|v or gate|up), shard each over ``world``
    ranks and concatenate this rank's pieces, so every rank holds its slice of every section. A section with
    fewer ``groups`` than ranks (K/V heads under a tensor-parallel size above their number) is replicated: rank
    ``r`` takes group ``r * groups // world``."""
    if world == 1:
        return w
    parts = []
    for i, piece in enumerate(torch.split(w, list(sections), dim=dim)):
        g = groups[i] if groups else None
        if g and g < world:
            if world % g or piece.shape[dim] % g:
                raise ValueError(f"section of {g} groups cannot be replicated over {world} ranks")
            parts.append(piece.chunk(g, dim=dim)[rank * g // world])
            continue
        if piece.shape[dim] % world != 0:
            raise ValueError(f"section of size {piece.shape[dim]} is not divisible by {world}")
        parts.append(piece.chunk(world, dim=dim)[rank])
    return torch.cat(parts, dim=dim).contiguous()


def _init_weight(shape, init_method, dtype, device, partition_dim=None, full_shape=None, rank=0, world=1,
                 sections=None, groups=None):
    """Initialise the full matrix with a fixed generator state, then keep this rank's slice, so the
    values do not depend on the tensor-parallel size."""
    w = torch.empty(full_shape or shape, dtype=torch.float32, device=device)
    init_method(w)
    if world > 1 and partition_dim is not None:
        if sections:
            w = shard_sections(w, sections, partition_dim, rank, world, groups)
        else:
            w = w.chunk(world, dim=partition_dim)[rank].contiguous()
    return nn.Parameter(w.to(dtype=dtype))


def _mark_tp(param, is_parallel, dim):
    param.tensor_model_parallel = is_parallel
    param.partition_dim = dim if is_parallel else -1
    param.partition_stride = 1


def default_init(std=0.02):
    from ..init_method import init_method_normal
    return init_method_normal(std)


class VocabParallelEmbedding(nn.Module):
    """Embedding table sharded over the vocabulary; out-of-shard ids give zero rows that the
    all-reduce (or reduce-scatter under sequence parallelism) fills in."""

    def __init__(self, num_embeddings: int, embedding_dim: int, *, config, init_method: Callable = None,
                 reduce_scatter_embeddings: bool = False):
        super().__init__()
        self.tp = ps.get_tensor_model_parallel_world_size()
        self.rank = ps.get_tensor_model_parallel_rank()
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.reduce_scatter_embeddings = reduce_scatter_embeddings
        per = math.ceil(num_embeddings / self.tp)
        self.vocab_start = self.rank * per
        self.vocab_end = min(num_embeddings, self.vocab_start + per)
        self.padded_rows = per
        dev = getattr(config, "device", None) or ("cuda" if torch.cuda.is_available() else "cpu")
        init = init_method or default_init(config.init_method_std)
        full = torch.zeros((per * self.tp, embedding_dim), dtype=torch.float32, device=dev)
        init(full[:num_embeddings])
        self.weight = nn.Parameter(full[self.vocab_start:self.vocab_start + per].to(dtype=config.params_dtype))
        _mark_tp(self.weight, self.tp > 1, 0)

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        flat = input_ids.reshape(-1)
        out = Fn.embedding(flat, self.weight, self.vocab_start)
        if self.tp > 1:
            if self.reduce_scatter_embeddings:
                out = M.reduce_scatter_to_sequence_parallel_region(out)
            else:
                out = M.reduce_from_tensor_model_parallel_region(out)
        return out


class _Fp8WeightMixin:
    """Inference-time block-scaled fp8 weights (DeepSeek-V3 checkpoint format: e4m3 values with one fp32
    ``weight_scale_inv`` per 128 x 128 block, reference ``toolkit/weight_convert/deepseekv3`` ``weight_dequant``).

    ``quantize_fp8_()`` replaces the bf16 parameter by the buffers ``weight_fp8`` / ``weight_scale_inv``;
    ``load_fp8_(w, s)`` installs checkpoint tensors directly. ``_mm`` then runs the fp8 GEMM with activations
    quantised per 1 x 128 block on the fly. Output rows that do not fill the last 128-row block are padded with zero
    rows (the checkpoint format does the same: its scale grid has ``ceil(rows / 128)`` entries) and the padding columns
    of the result are sliced off; layers whose input width is not a multiple of 128 stay in bf16.
    """
    weight_fp8 = None
    weight_scale_inv = None
    _fp8_rows = None          # true number of output rows when ``weight_fp8`` carries padding rows

    def quantize_fp8_(self) -> bool:
        w = self.weight
        if w is None or w.dim() != 2 or w.shape[0] % 8 or w.shape[1] % 128:
            return False
        wq, scale = Fn.quantize_weight_128x128(_pad_rows_128(w.detach()))
        return self.load_fp8_(wq, scale, rows=w.shape[0])

    def load_fp8_(self, wq: torch.Tensor, scale_inv: torch.Tensor, rows: Optional[int] = None) -> bool:
        rows = wq.shape[0] if rows is None else rows
        self._parameters.pop("weight", None)
        self.weight = None
        self.weight_fp8 = _pad_rows_128(wq)
        self.weight_scale_inv = scale_inv.float().contiguous()
        self._fp8_rows = rows if rows != self.weight_fp8.shape[0] else None
        return True

    def _mm(self, x: torch.Tensor, w: Optional[torch.Tensor] = None) -> torch.Tensor:
        if w is None and self.weight_fp8 is not None:
            y = Fn.fp8_linear(x, self.weight_fp8, self.weight_scale_inv)
            return y if self._fp8_rows is None else y[..., :self._fp8_rows]
        return Fn.linear(x, self.weight if w is None else w)


def _pad_rows_128(w: torch.Tensor) -> torch.Tensor:
    """``w [N, K]`` with zero rows appended up to the next multiple of 128 (no copy when N already is one)."""
    pad = -w.shape[0] % 128
    if pad == 0:
        return w
    out = torch.zeros(w.shape[0] + pad, w.shape[1], dtype=w.dtype, device=w.device)
    out[:w.shape[0]] = w
    return out


class ColumnParallelLinear(_Fp8WeightMixin, nn.Module):
    """``Y = X W^T`` with ``W`` split along its output rows."""

    def __init__(self, input_size: int, output_size: int, *, config, init_method: Callable = None,
                 bias: bool = False, gather_output: bool = False, skip_bias_add: bool = False,
                 skip_weight_param_allocation: bool = False, is_expert: bool = False, tp_group=None,
                 stride: int = 1, partition_sections=None, partition_groups=None):
        super().__init__()
        self.config = config
        self.tp = 1 if is_expert and config.expert_tensor_parallel_size == 1 else ps.get_tensor_model_parallel_world_size()
        self.rank = ps.get_tensor_model_parallel_rank() if self.tp > 1 else 0
        self.input_size, self.output_size = input_size, output_size
        if partition_sections and partition_groups and self.tp > 1:
            # sections with fewer groups than ranks (K/V heads) are replicated, so a rank holds more than 1/tp of the rows
            self.output_size_per_partition = sum(section_local_sizes(partition_sections, self.tp, partition_groups))
        else:
            partition_groups = None
            if output_size % self.tp != 0:
                raise ValueError(f"output_size {output_size} is not divisible by the tensor-parallel size {self.tp}")
            self.output_size_per_partition = output_size // self.tp
        self.gather_output, self.skip_bias_add = gather_output, skip_bias_add
        self.sequence_parallel = bool(config.sequence_parallel) and self.tp > 1
        self.is_expert = is_expert
        dev = getattr(config, "device", None) or ("cuda" if torch.cuda.is_available() else "cpu")
        init = init_method or default_init(config.init_method_std)
        if skip_weight_param_allocation:
            self.weight = None
        else:
            self.weight = _init_weight((self.output_size_per_partition, input_size), init, config.params_dtype, dev,
                                       partition_dim=0, full_shape=(output_size, input_size), rank=self.rank,
                                       world=self.tp, sections=partition_sections, groups=partition_groups)
            _mark_tp(self.weight, self.tp > 1, 0)
            self.weight.partition_stride = stride
            self.weight.partition_sections = tuple(partition_sections) if partition_sections else None
            self.weight.partition_groups = tuple(partition_groups) if partition_groups else None
        if bias:
            self.bias = nn.Parameter(torch.zeros(self.output_size_per_partition, dtype=config.params_dtype, device=dev))
            _mark_tp(self.bias, self.tp > 1, 0)
            self.bias.partition_sections = tuple(partition_sections) if partition_sections else None
            self.bias.partition_groups = tuple(partition_groups) if partition_groups else None
        else:
            self.register_parameter("bias", None)

    def forward(self, x: torch.Tensor, weight: Optional[torch.Tensor] = None):
        w = self.weight if weight is None else weight
        fp8 = weight is None and self.weight_fp8 is not None
        bias = None if self.skip_bias_add else self.bias
        if self.tp > 1:
            if self.sequence_parallel:
                from .. import fused_comm
                if not fp8 and fused_comm.enabled(self.config, x):
                    y = fused_comm.allgather_linear(x, w)
                else:
                    y = self._mm(M.gather_from_sequence_parallel_region(x), weight)
            else:
                y = self._mm(M.copy_to_tensor_model_parallel_region(x), weight)
        else:
            y = self._mm(x, weight)
        if bias is not None:
            y = y + bias
        if self.gather_output and self.tp > 1:
            y = M.gather_from_tensor_model_parallel_region(y)
        return y, (self.bias if self.skip_bias_add else None)


class RowParallelLinear(_Fp8WeightMixin, nn.Module):
    """``Y = X W^T`` with ``W`` split along its input columns; partial sums are reduced over TP."""

    def __init__(self, input_size: int, output_size: int, *, config, init_method: Callable = None,
                 bias: bool = False, input_is_parallel: bool = True, skip_bias_add: bool = False,
                 is_expert: bool = False, delay_allreduce: bool = False):
        super().__init__()
        self.config = config
        self.tp = 1 if is_expert and config.expert_tensor_parallel_size == 1 else ps.get_tensor_model_parallel_world_size()
        self.rank = ps.get_tensor_model_parallel_rank() if self.tp > 1 else 0
        if input_size % self.tp != 0:
            raise ValueError(f"input_size {input_size} is not divisible by the tensor-parallel size {self.tp}")
        self.input_size, self.output_size = input_size, output_size
        self.input_size_per_partition = input_size // self.tp
        self.input_is_parallel, self.skip_bias_add = input_is_parallel, skip_bias_add
        self.sequence_parallel = bool(config.sequence_parallel) and self.tp > 1
        self.delay_allreduce = delay_allreduce
        dev = getattr(config, "device", None) or ("cuda" if torch.cuda.is_available() else "cpu")
        init = init_method or default_init(config.output_layer_init_std)
        self.weight = _init_weight((output_size, self.input_size_per_partition), init, config.params_dtype, dev,
                                   partition_dim=1, full_shape=(output_size, input_size), rank=self.rank,
                                   world=self.tp)
        _mark_tp(self.weight, self.tp > 1, 1)
        if bias:
            self.bias = nn.Parameter(torch.zeros(output_size, dtype=config.params_dtype, device=dev))
            _mark_tp(self.bias, False, -1)
            self.bias.sequence_parallel = self.sequence_parallel
        else:
            self.register_parameter("bias", None)

    def forward(self, x: torch.Tensor):
        if not self.input_is_parallel and self.tp > 1:
            x = x.chunk(self.tp, dim=-1)[self.rank].contiguous()
        fp8 = self.weight_fp8 is not None
        if self.tp > 1 and not self.delay_allreduce:
            from .. import fused_comm
            if self.sequence_parallel:
                if not fp8 and fused_comm.enabled(self.config, x):
                    y = fused_comm.linear_reduce_scatter(x, self.weight)
                else:
                    y = M.reduce_scatter_to_sequence_parallel_region(self._mm(x))
            else:
                if not fp8 and fused_comm.allreduce_enabled(self.config, x, self.weight):
                    y = fused_comm.linear_all_reduce(x, self.weight)      # inference: GEMM -> all-reduce in one kernel
                else:
                    y = self._mm(x)
                    from .. import ll_allreduce
                    group = ps.get_tensor_model_parallel_group()
                    if getattr(self.config, "fused_tp_comm", False) and ll_allreduce.usable(group, y):
                        # decode-sized output (also of fp8 layers, also under CUDA-graph capture): one launch in which
                        # the data carries its own arrival
                        y = ll_allreduce.get(group)(y, out=y)
                    else:
                        y = M.reduce_from_tensor_model_parallel_region(y)
        else:
            y = self._mm(x)
        if self.bias is not None and not self.skip_bias_add:
            y = y + self.bias
        return y, (self.bias if self.skip_bias_add else None)


class LinearNoTP(_Fp8WeightMixin, nn.Module):
    """Replicated linear layer (the reference's ``LinearNoTP`` / ``ReplicatedLinear``)."""

    def __init__(self, input_size: int, output_size: int, *, config, init_method: Callable = None,
                 bias: bool = False, skip_bias_add: bool = False, params_dtype=None):
        super().__init__()
        self.config = config
        self.skip_bias_add = skip_bias_add
        dev = getattr(config, "device", None) or ("cuda" if torch.cuda.is_available() else "cpu")
        init = init_method or default_init(config.init_method_std)
        dtype = params_dtype or config.params_dtype
        self.weight = _init_weight((output_size, input_size), init, dtype, dev)
        _mark_tp(self.weight, False, -1)
        self.weight.sequence_parallel = bool(config.sequence_parallel)
        if bias:
            self.bias = nn.Parameter(torch.zeros(output_size, dtype=dtype, device=dev))
            self.bias.sequence_parallel = bool(config.sequence_parallel)
        else:
            self.register_parameter("bias", None)

    def forward(self, x):
        y = self._mm(x)
        if self.bias is not None and not self.skip_bias_add:
            y = y + self.bias
        return y, (self.bias if self.skip_bias_add else None)


ReplicatedLinear = LinearNoTP


class ColumnParallelBatchedLinear(nn.Module):
    """One column-parallel linear per expert, applied as a batched product: ``x [E_local, C, in]`` (the capacity-based
    expert layout: C token slots per expert) times ``weight [E_local, out / etp, in]``. Experts are split over the
    expert-parallel group (axis 0) and every expert's output rows over the expert-tensor-parallel group.

    Reference: ``training_graph/tensor_parallel/batched_layers.py:29-226`` (``ColumnParallelBatchedLinear``)."""

    def __init__(self, input_size: int, output_size: int, *, config, init_method: Callable = None,
                 bias: bool = False, skip_bias_add: bool = False, is_expert: bool = True):
        super().__init__()
        if not is_expert or not config.num_moe_experts or config.num_moe_experts < 2:
            raise ValueError("batched linears are expert layers: is_expert=True and num_moe_experts > 1 are required")
        if bias:
            raise ValueError("batched expert linears carry no bias")
        ep, etp = ps.get_expert_model_parallel_world_size(), ps.get_expert_tensor_parallel_world_size()
        E = config.num_moe_experts
        if E % ep or output_size % etp:
            raise ValueError(f"experts {E} / output rows {output_size} do not split over ep {ep} / etp {etp}")
        self.config, self.num_local_experts = config, E // ep
        dev = getattr(config, "device", None) or ("cuda" if torch.cuda.is_available() else "cpu")
        init = init_method or default_init(config.init_method_std)
        full = torch.empty(E, output_size, input_size, dtype=torch.float32, device=dev)
        init(full)                                       # whole stack first: values do not depend on ep / etp
        er, tr = ps.get_expert_model_parallel_rank(), ps.get_expert_tensor_parallel_rank()
        local = full[er * self.num_local_experts:(er + 1) * self.num_local_experts]
        local = local.chunk(etp, dim=1)[tr].contiguous()
        self.weight = nn.Parameter(local.to(config.params_dtype))
        self.weight.is_expert = True
        _mark_tp(self.weight, etp > 1, 1)

    def forward(self, x: torch.Tensor, weight: Optional[torch.Tensor] = None):
        w = self.weight if weight is None else weight
        y = torch.bmm(x.to(w.dtype), w.transpose(1, 2))
        return y.to(x.dtype), None


class RowParallelBatchedLinear(nn.Module):
    """Per-expert row-parallel linear: ``x [E_local, C, in / etp]`` times ``weight [E_local, out, in / etp]``, partial
    sums all-reduced over the expert-tensor-parallel group.

    Reference: ``training_graph/tensor_parallel/batched_layers.py:228-399`` (``RowParallelBatchedLinear``)."""

    def __init__(self, input_size: int, output_size: int, *, config, init_method: Callable = None,
                 bias: bool = False, skip_bias_add: bool = False, is_expert: bool = True):
        super().__init__()
        if not is_expert or not config.num_moe_experts or config.num_moe_experts < 2:
            raise ValueError("batched linears are expert layers: is_expert=True and num_moe_experts > 1 are required")
        if bias:
            raise ValueError("batched expert linears carry no bias")
        ep, etp = ps.get_expert_model_parallel_world_size(), ps.get_expert_tensor_parallel_world_size()
        E = config.num_moe_experts
        if E % ep or input_size % etp:
            raise ValueError(f"experts {E} / input columns {input_size} do not split over ep {ep} / etp {etp}")
        self.config, self.num_local_experts, self.etp = config, E // ep, etp
        dev = getattr(config, "device", None) or ("cuda" if torch.cuda.is_available() else "cpu")
        init = init_method or default_init(config.output_layer_init_std)
        full = torch.empty(E, output_size, input_size, dtype=torch.float32, device=dev)
        init(full)
        er, tr = ps.get_expert_model_parallel_rank(), ps.get_expert_tensor_parallel_rank()
        local = full[er * self.num_local_experts:(er + 1) * self.num_local_experts]
        local = local.chunk(etp, dim=2)[tr].contiguous()
        self.weight = nn.Parameter(local.to(config.params_dtype))
        self.weight.is_expert = True
        _mark_tp(self.weight, etp > 1, 2)

    def forward(self, x: torch.Tensor):
        y = torch.bmm(x.to(self.weight.dtype), self.weight.transpose(1, 2))
        if self.etp > 1:
            y = _AllReduceSum.apply(y, ps.get_expert_tensor_parallel_group())
        return y.to(x.dtype), None


class _AllReduceSum(torch.autograd.Function):
    """Sum over a group in forward, identity in backward (every rank holds the full gradient of the sum)."""

    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous()
        torch.distributed.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None
