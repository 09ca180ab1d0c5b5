"""``MicroBatchInterleaved``: a batch split into copies whose forward passes are issued on separate CUDA streams.

Reference: ``trainer/base_trainer.py:496-498`` wraps the network in MindSpore's ``MicroBatchInterleaved(net, n)``
(``micro_batch_interleave_num``) so that the tensor-parallel collectives of one half of the batch overlap the
matrix products of the other half. Here the copies run on their own streams: kernels of different copies may overlap,
in particular a copy's NCCL collective with the other copy's GEMMs. The fused GEMM + collective kernels already
overlap both inside one kernel, so this wrapper matters for the paths that still call NCCL (fp8 layers, pipeline
stages). The loss is the mean of the copies' losses, which equals the loss of the whole batch when every copy has the
same number of loss tokens; with ``(numerator, denominator)`` losses the parts are summed.
"""
from __future__ import annotations

from typing import Any, Dict

import torch
import torch.nn as nn


def _split(value: Any, n: int, batch: int):
    if isinstance(value, torch.Tensor) and value.dim() >= 1 and value.shape[0] == batch:
        return list(value.chunk(n, dim=0))
    return [value] * n


class MicroBatchInterleaved(nn.Module):
    """Wraps a network: the batch is cut into ``interleave_num`` copies along dimension 0, each runs on its own CUDA
    stream, scalar losses are averaged, ``(numerator, denominator)`` losses summed, other tensors concatenated."""

    def __init__(self, network: nn.Module, interleave_num: int = 2):
        super().__init__()
        if interleave_num < 1:
            raise ValueError("interleave_num must be at least 1")
        self.network, self.interleave_num = network, int(interleave_num)
        self._streams = None

    def forward(self, *args, **kwargs):
        n = self.interleave_num
        first = next((a for a in list(args) + list(kwargs.values()) if isinstance(a, torch.Tensor) and a.dim() >= 1), None)
        if n == 1 or first is None:
            return self.network(*args, **kwargs)
        batch = first.shape[0]
        if batch % n:
            raise ValueError(f"batch size {batch} is not divisible by micro_batch_interleave_num {n}")
        arg_parts = [_split(a, n, batch) for a in args]
        kw_parts: Dict[str, list] = {k: _split(v, n, batch) for k, v in kwargs.items()}
        use_streams = first.is_cuda
        if use_streams and self._streams is None:
            self._streams = [torch.cuda.Stream(device=first.device) for _ in range(n)]
        outs = []
        cur = torch.cuda.current_stream(first.device) if use_streams else None
        for i in range(n):
            a_i = [p[i] for p in arg_parts]
            k_i = {k: p[i] for k, p in kw_parts.items()}
            if use_streams:
                self._streams[i].wait_stream(cur)
                with torch.cuda.stream(self._streams[i]):
                    outs.append(self.network(*a_i, **k_i))
            else:
                outs.append(self.network(*a_i, **k_i))
        if use_streams:
            for st in self._streams:
                cur.wait_stream(st)
        return self._merge(outs)

    @staticmethod
    def _merge(outs):
        head = outs[0]
        if isinstance(head, tuple):                     # (numerator, denominator, ...) style losses: sum the parts
            return tuple(sum(o[j] for o in outs) for j in range(len(head)))
        if isinstance(head, torch.Tensor) and head.dim() == 0:
            return sum(outs) / len(outs)
        if isinstance(head, torch.Tensor):
            return torch.cat(outs, dim=0)
        return outs
