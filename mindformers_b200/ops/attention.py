"""Front-end of the hand-written flash-attention kernels (``csrc/flash_attention.cu``)."""
from __future__ import annotations

import torch

from . import _lib


def supported(q, k, v, causal) -> bool:
    """True when the native kernel covers this problem (bf16, head dim 128, equal q/k lengths)."""
    lib = _lib.get_lib()
    return hasattr(lib, "mfb_flash_attn_fwd") and _shape_ok(q, k, v)


def _shape_ok(q, k, v) -> bool:
    return (q.dtype == torch.bfloat16 and q.shape[-1] == 128 and v.shape[-1] == 128
            and q.shape[1] == k.shape[1] and q.shape[1] % 128 == 0 and q.shape[2] % k.shape[2] == 0)


def flash_attention(q, k, v, causal=True, scale=None):
    raise _lib.KernelLibraryError("flash attention kernel is not part of this build")
