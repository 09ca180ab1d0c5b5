"""Flat parameter / gradient buffers.

Every parameter of a model chunk becomes a view into one flat buffer per (dtype, reduction group), and
gets a ``main_grad`` view into a flat fp32 (or bf16) gradient buffer that the wgrad kernels accumulate
into. This is what lets the data-parallel reduce-scatter, the fused AdamW kernel and the parameter
all-gather each run as a single pass over contiguous memory (the mechanism behind the reference's
``parallel.enable_parallel_optimizer`` / ``optimizer_shard``, which MindSpore implements internally).

Order inside a buffer (so that weight decay, the TP-replicated set and the set needing a TP all-reduce
are each one contiguous range):
    [sharded, decay] [replicated, decay] [replicated+SP-reduced, decay]
    [replicated+SP-reduced, no decay] [replicated, no decay] [sharded, no decay]
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

ALIGN = 128  # elements; keeps every parameter 256-byte aligned for TMA and vector accesses


def _no_decay(name: str, p: torch.Tensor) -> bool:
    if getattr(p, "no_weight_decay", False):
        return True
    return p.dim() <= 1 or name.endswith(".bias")


def _category(name: str, p: torch.Tensor, tp: int, sequence_parallel: bool) -> int:
    nd = _no_decay(name, p)
    sharded = bool(getattr(p, "tensor_model_parallel", False)) or tp == 1 or getattr(p, "is_expert", False)
    sp_reduce = (not sharded) and sequence_parallel and bool(getattr(p, "sequence_parallel", False))
    if sharded:
        return 5 if nd else 0
    if sp_reduce:
        return 3 if nd else 2
    return 4 if nd else 1


@dataclass
class BufferRanges:
    """Where a parameter sits inside a flat bucket buffer and which slice of the bucket each data-parallel rank owns."""

    numel: int = 0            # padded to a multiple of pad_to
    decay_end: int = 0        # [0, decay_end) gets weight decay
    dup_begin: int = 0        # [dup_begin, dup_end) is replicated over tensor-parallel ranks
    dup_end: int = 0
    sp_begin: int = 0         # [sp_begin, sp_end) needs a gradient all-reduce over the TP group
    sp_end: int = 0


class ParamAndGradBuffer:
    """One flat parameter buffer + gradient buffer for a list of named parameters."""

    def __init__(self, named_params: List[Tuple[str, torch.nn.Parameter]], *, tp: int = 1,
                 sequence_parallel: bool = False, grad_dtype: torch.dtype = torch.float32, pad_to: int = 1,
                 name: str = "dense", allocator=None):
        self.name = name
        if not named_params:
            raise ValueError("empty parameter list")
        dtype = named_params[0][1].dtype
        device = named_params[0][1].device
        if any(p.dtype != dtype for _, p in named_params):
            raise ValueError("all parameters of a buffer must share one dtype")
        cats = [(_category(n, p, tp, sequence_parallel), i) for i, (n, p) in enumerate(named_params)]
        order = [i for _, i in sorted(cats, key=lambda c: (c[0], c[1]))]
        self.entries: List[Tuple[str, torch.nn.Parameter, int, int]] = []
        off = 0
        bounds = {c: [None, None] for c in range(6)}
        for i in order:
            n, p = named_params[i]
            c = cats[i][0]
            if bounds[c][0] is None:
                bounds[c][0] = off
            self.entries.append((n, p, off, p.numel()))
            off += (p.numel() + ALIGN - 1) // ALIGN * ALIGN
            bounds[c][1] = off
        step = ALIGN * max(pad_to, 1)
        total = (off + step - 1) // step * step

        def begin(cs, default):
            vals = [bounds[c][0] for c in cs if bounds[c][0] is not None]
            return min(vals) if vals else default

        def end(cs, default):
            vals = [bounds[c][1] for c in cs if bounds[c][1] is not None]
            return max(vals) if vals else default

        r = BufferRanges(numel=total)
        r.decay_end = end((0, 1, 2), 0)
        r.dup_begin, r.dup_end = begin((1, 2, 3, 4), 0), end((1, 2, 3, 4), 0)
        r.sp_begin, r.sp_end = begin((2, 3), 0), end((2, 3), 0)
        self.ranges = r
        # ``allocator(tag, numel, dtype, device)`` lets the optimizer place the buffers in peer-mapped memory
        alloc = allocator or (lambda tag, numel, dt, dev: torch.zeros(numel, dtype=dt, device=dev))
        self.param_data = alloc(f"{name}.param", total, dtype, device)
        self.grad_data = alloc(f"{name}.grad", total, grad_dtype, device)
        self.index: Dict[str, Tuple[int, int, torch.Size]] = {}
        for n, p, o, cnt in self.entries:
            view = self.param_data[o:o + cnt].view(p.shape)
            view.copy_(p.data)
            p.data = view
            p.main_grad = self.grad_data[o:o + cnt].view(p.shape)
            self.index[n] = (o, cnt, p.shape)

    def zero_grad(self):
        self.grad_data.zero_()

    def collect_autograd_grads(self):
        """Fold ``.grad`` tensors produced by ordinary autograd paths into ``main_grad`` and drop them."""
        for _, p, _, _ in self.entries:
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                p.grad = None


def build_buffers(model: torch.nn.Module, *, tp: int, sequence_parallel: bool, grad_dtype=torch.float32,
                  dense_pad: int = 1, expert_pad: int = 1, allocator=None) -> Dict[str, ParamAndGradBuffer]:
    """Split trainable parameters into the dense and the expert buffer (they reduce over different groups)."""
    dense, expert = [], []
    for n, p in model.named_parameters():
        if not p.requires_grad:
            continue
        (expert if getattr(p, "allreduce", True) is False else dense).append((n, p))
    out = {}
    groups = (("dense", dense, dense_pad), ("expert", expert, expert_pad))
    for key, plist, pad in groups:
        by_dtype: Dict[torch.dtype, list] = {}
        for n, p in plist:
            by_dtype.setdefault(p.dtype, []).append((n, p))
        for dt, lst in by_dtype.items():
            name = key if len(by_dtype) == 1 else f"{key}_{str(dt).replace('torch.', '')}"
            out[name] = ParamAndGradBuffer(lst, tp=tp, sequence_parallel=sequence_parallel, grad_dtype=grad_dtype,
                                           pad_to=pad, name=name, allocator=allocator)
    return out
