"""Fused compute + collective paths over NVLink peer memory (front-end).

``enabled`` / ``moe_enabled`` decide per call whether the fused kernels can serve it; otherwise the
layers fall back to the NCCL collectives of ``mappings``. The kernels themselves live in
``ops/csrc/fused_comm.cu`` and work on symmetric buffers registered through ``parallel/symm_mem.py``.
"""
from __future__ import annotations

import torch

from . import parallel_state as ps

_FORCE_OFF = False


def set_enabled(flag: bool):
    """Global switch (the NCCL baseline of the benchmark turns the fused paths off)."""
    global _FORCE_OFF
    _FORCE_OFF = not flag


def dp_enabled() -> bool:
    """Fused data-parallel optimizer path (reduce-scatter by peer loads, AdamW, all-gather by peer stores)."""
    import os
    return not _FORCE_OFF and torch.cuda.is_available() and os.environ.get("MFB_FUSED_DP", "1") != "0"


def cp_enabled() -> bool:
    """Context-parallel K/V exchange through the peer-memory kernels (``parallel/fused_cp.py``)."""
    import os
    return not _FORCE_OFF and torch.cuda.is_available() and os.environ.get("MFB_FUSED_CP", "1") != "0"


def _runtime_ready() -> bool:
    from . import symm_mem
    return symm_mem.is_ready()


def enabled(config, x: torch.Tensor) -> bool:
    """True when the fused tensor-parallel kernels can serve this call (bf16 on CUDA, token count a
    multiple of 128 per rank); the layers fall back to NCCL collectives + GEMM otherwise."""
    if _FORCE_OFF or not getattr(config, "fused_tp_comm", False) or not x.is_cuda:
        return False
    tp = ps.get_tensor_model_parallel_world_size()
    if tp == 1 or x.dtype != torch.bfloat16 or x.dim() != 2:
        return False
    return x.shape[0] % 128 == 0 and x.shape[1] % 64 == 0


def allreduce_enabled(config, x: torch.Tensor, weight: torch.Tensor) -> bool:
    """True when the one-shot GEMM -> all-reduce kernel can serve a row-parallel layer without sequence parallelism
    (tensor-parallel inference): bf16 on CUDA, no gradient needed, at most ``fused_tp.AR_MAX_ROWS`` tokens."""
    if _FORCE_OFF or not getattr(config, "fused_tp_comm", False) or not x.is_cuda or x.dim() != 2:
        return False
    if ps.get_tensor_model_parallel_world_size() == 1 or x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        return False
    if torch.is_grad_enabled() and (x.requires_grad or weight.requires_grad):
        return False
    if torch.cuda.is_current_stream_capturing():
        return False            # the kernel's flag epoch comes from the host: a replay would reuse it
    from . import fused_tp
    return fused_tp.allreduce_shapes_ok(x.shape[0], x.shape[1], weight.shape[0])


def moe_enabled(config, x: torch.Tensor) -> bool:
    """True when the device-side MoE exchange (``parallel/fused_moe.py``) can serve this call: bf16 on CUDA,
    any expert-parallel size up to 8 (size 1 = local permute kernels)."""
    if _FORCE_OFF or not getattr(config, "fused_moe_comm", False) or not x.is_cuda:
        return False
    from . import fused_moe
    return fused_moe.supported(config, x)


def allgather_linear(x, w):
    from . import fused_tp
    return fused_tp.allgather_linear(x, w)


def linear_reduce_scatter(x, w):
    from . import fused_tp
    return fused_tp.linear_reduce_scatter(x, w)


def linear_all_reduce(x, w):
    from . import fused_tp
    return fused_tp.gemm_all_reduce(x, w)


def moe_dispatch_experts_combine(layer, hidden, probs, ids):
    from . import fused_moe
    return fused_moe.moe_dispatch_experts_combine(layer, hidden, probs, ids)
