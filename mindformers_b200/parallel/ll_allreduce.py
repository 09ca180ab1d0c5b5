"""Low-latency all-reduce of small bf16 tensors over NVLink peer memory (``ops/csrc/ll_allreduce.cu``).

The reference's tensor-parallel inference layers reduce the row-parallel output with an all-reduce after every
attention and MLP block (``parallel_core/inference/tensor_parallel/layers.py:373-407``,
``inference/tensor_parallel/mappings.py``); at decode sizes that collective is pure latency. This one is a single
launch in which the data carries its own arrival (sentinel-filled receive buffers, three rotating generations), the
call counter lives on the device, and the sum is taken in rank order, so every rank gets the same bits and the launch
can be captured in a CUDA graph.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..ops import _lib
from . import symm_mem

MAX_BYTES = int(os.environ.get("MFB_LL_ALLREDUCE_MAX_BYTES", str(2 * 1024 * 1024)))
_ENABLED = os.environ.get("MFB_LL_ALLREDUCE", "1") != "0"
_INSTANCES: Dict[int, "LLAllReduce"] = {}


def set_enabled(flag: bool) -> None:
    global _ENABLED
    _ENABLED = bool(flag)


class LLAllReduce:
    """Receive buffers, peer pointer table and device-side call counter of one process group (at most 8 ranks)."""

    def __init__(self, group, device=None, max_bytes: int = MAX_BYTES):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > 8:
            raise ValueError("the low-latency all-reduce serves at most 8 ranks")
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.max_bytes = int(max_bytes)
        lib = _lib.get_lib()
        nbytes = int(lib.mfb_ll_allreduce_buffer_bytes(self.world, self.max_bytes))
        self.buf = symm_mem.allocate(f"ll_allreduce.{self.max_bytes}", nbytes, group, self.device)
        self.ptrs = (ctypes.c_longlong * self.world)(*[int(p) for p in self.buf.ptrs])
        self.state = torch.zeros(int(lib.mfb_ll_allreduce_state_words()), dtype=torch.int32, device=self.device)
        _lib.check(lib.mfb_ll_allreduce_init(self.buf.tensor.data_ptr(), nbytes, _lib.stream_ptr()), "mfb_ll_allreduce_init")
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)           # every rank's buffer holds the sentinel before anyone sends

    def supports(self, x: torch.Tensor) -> bool:
        n = x.numel() * x.element_size()
        return x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and 0 < n <= self.max_bytes and n % 16 == 0 \
            and x.data_ptr() % 16 == 0

    def __call__(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Sum of ``x`` over the ranks of the group (same bits on every rank). ``out`` may be ``x`` itself."""
        if not self.supports(x):
            raise ValueError("ll_allreduce: a contiguous, 16-byte aligned bf16 CUDA tensor of at most "
                             f"{self.max_bytes} bytes (a multiple of 16) is required")
        out = torch.empty_like(x) if out is None else out
        rc = _lib.get_lib().mfb_ll_allreduce(x.data_ptr(), out.data_ptr(), x.numel() * 2, self.max_bytes, self.world, self.rank,
                                             self.ptrs, self.state.data_ptr(), _lib.status_word(x.device).data_ptr(),
                                             _lib.stream_ptr())
        _lib.check(rc, "mfb_ll_allreduce")
        _lib.count_launch(1)
        return out


def get(group) -> LLAllReduce:
    """The instance of ``group`` (created by the first call: a collective, every rank of the group must make it at the
    same point of the program, outside a CUDA-graph capture)."""
    inst = _INSTANCES.get(id(group))
    if inst is None:
        inst = _INSTANCES[id(group)] = LLAllReduce(group)
    return inst


def usable(group, x: torch.Tensor) -> bool:
    """Whether ``all_reduce(x)`` over ``group`` can take the low-latency kernel now. The decision depends on shapes
    and settings only (never on timing), so every rank of the group takes the same one."""
    if not _ENABLED or group is None or not x.is_cuda or x.dtype != torch.bfloat16:
        return False
    if torch.is_grad_enabled() and x.requires_grad:
        return False
    n = x.numel() * 2
    if n == 0 or n > MAX_BYTES or n % 16 or not x.is_contiguous() or x.data_ptr() % 16:
        return False
    if dist.get_world_size(group) > 8 or dist.get_world_size(group) < 2:
        return False
    if id(group) not in _INSTANCES and torch.cuda.is_current_stream_capturing():
        return False            # the set-up is a host collective: it cannot happen inside a capture
    return True
