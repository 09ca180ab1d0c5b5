"""Symmetric (peer-mapped) device buffers for the fused communication kernels.

Built on ``torch.distributed._symmetric_memory``: every rank allocates the same buffer, the rendezvous
exchanges handles, and each rank gets the table of peer base pointers (plain P2P loads/stores over
NVLink), the multicast pointer when NVLS is available, and a signal pad for flags.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

_BUFFERS: Dict[str, object] = {}
_READY = False


def is_ready() -> bool:
    return _READY


class SymmBuffer:
    """A peer-mapped allocation: the local tensor, the device pointers of the same buffer on every rank of the group
    (``ptrs``) and the handle that keeps the mapping alive."""

    def __init__(self, tensor, handle):
        self.tensor = tensor
        self.handle = handle
        self.world = handle.world_size
        self.rank = handle.rank
        # torch sub-allocates symmetric tensors from pooled blocks: ``buffer_ptrs`` are the block bases on every
        # rank and ``offset`` is where this tensor starts inside its block (the same on all ranks)
        off = int(getattr(handle, "offset", 0) or 0)
        self.offset = off
        self.ptrs = [int(p) + off for p in handle.buffer_ptrs]
        if self.ptrs[self.rank] != tensor.data_ptr():
            raise RuntimeError(f"symmetric buffer: local address {tensor.data_ptr():#x} is not block base + offset "
                               f"({self.ptrs[self.rank]:#x}); peer pointers cannot be derived")
        self.peer_ptrs = torch.tensor(self.ptrs, dtype=torch.int64, device=tensor.device)
        self.signal_ptrs = torch.tensor(list(handle.signal_pad_ptrs), dtype=torch.int64, device=tensor.device)
        mc = int(getattr(handle, "multicast_ptr", 0) or 0)
        self.multicast_ptr = mc + off if mc else 0


def allocate(name: str, nbytes: int, group, device=None) -> SymmBuffer:
    """Allocate (once per name) a symmetric byte buffer shared by the ranks of ``group``."""
    global _READY
    import torch.distributed._symmetric_memory as symm
    key = f"{name}:{id(group)}"
    buf = _BUFFERS.get(key)
    if buf is not None and buf.tensor.numel() >= nbytes:
        return buf
    device = device or torch.device("cuda", torch.cuda.current_device())
    t = symm.empty(nbytes, dtype=torch.uint8, device=device)
    h = symm.rendezvous(t, group=group)
    buf = SymmBuffer(t, h)
    _BUFFERS[key] = buf
    _READY = True
    return buf


def free(name: str, group) -> None:
    """Drop this module's reference to a buffer. Call it on every rank at the same point of the program, after a
    collective that orders all peers' reads of the buffer before it."""
    _BUFFERS.pop(f"{name}:{id(group)}", None)


def enable():
    global _READY
    _READY = True


def disable():
    global _READY
    _READY = False
