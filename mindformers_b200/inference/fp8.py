"""Block-scaled fp8 weights for inference.

``quantize_model_fp8(model)`` converts the linear layers and the grouped expert weights of a built model to e4m3
values with one fp32 scale per 128 x 128 block (the format of DeepSeek-V3 checkpoints; the reference only
de-quantises such checkpoints to bf16, ``toolkit/weight_convert/deepseekv3/convert_deepseekv3_hf_weight.py:67-114``).
The GEMMs then run on ``ops/csrc/gemm_fp8.cu`` with activations quantised per 1 x 128 block on the fly.

Kept in bf16: embeddings and the output layer, routers, norms, the MLA ``linear_kvb`` (decode reads its rows as the
absorbed up-projections) and every layer whose shape is not a multiple of 128.
"""
from __future__ import annotations

from typing import Dict, Iterable

import torch

DEFAULT_SKIP = ("output_layer", "embedding", "router", "linear_kvb")


def quantize_model_fp8(model: torch.nn.Module, skip: Iterable[str] = DEFAULT_SKIP) -> Dict[str, int]:
    """Returns ``{"linear": n, "grouped": n, "kept": n, "bytes_before": b, "bytes_after": b}``."""
    skip = tuple(skip)
    stats = {"linear": 0, "grouped": 0, "kept": 0, "bytes_before": 0, "bytes_after": 0}
    with torch.no_grad():
        for name, mod in model.named_modules():
            fn = getattr(mod, "quantize_fp8_", None)
            if fn is None:
                continue
            before = sum(p.numel() * p.element_size() for p in mod.parameters(recurse=False))
            if any(s in name for s in skip) or not fn():
                stats["kept"] += 1
                continue
            after = sum(p.numel() * p.element_size() for p in mod.parameters(recurse=False))
            for attr in ("weight_fp8", "weight_scale_inv", "w1_fp8", "w2_fp8", "w1_scale_inv", "w2_scale_inv"):
                t = getattr(mod, attr, None)
                if t is not None:
                    after += t.numel() * t.element_size()
            stats["bytes_before"] += before
            stats["bytes_after"] += after
            stats["grouped" if hasattr(mod, "w1_fp8") and mod.w1_fp8 is not None else "linear"] += 1
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
    return stats
