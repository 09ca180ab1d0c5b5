"""Parameter groups for optimizers that take ``torch.optim`` style groups (CAME, SGD, ...): which parameters are exempt
from weight decay, and optionally a learning rate that decays from the top layer down.

Reference: ``trainer/optimizer_grouped_parameters.py:29`` (``get_optimizer_grouped_parameters``: no decay for
one-dimensional parameters, biases and the names / keywords a model lists in ``no_weight_decay()`` /
``no_weight_decay_keywords()``; with ``layer_scale`` a per-layer factor ``layer_decay ** (num_layers + 1 - layer_id)``
on the learning rate, embedding = layer 0, decoder layer i = i + 1, everything after the decoder = num_layers + 1).
The sharded AdamW (``parallel/distributed/optimizer.py``) keeps its own decay ranges inside the flat buffers and has one
learning rate; groups from here feed ``core/optim.py::ReplicatedOptimizer``, which multiplies the scheduled learning
rate by each group's ``lr_scale``."""
from __future__ import annotations

import re
from typing import Dict, List, Optional

import torch

from ..tools.logger import logger

_LAYER = re.compile(r"(?:^|\.)layers\.(\d+)\.")


def _layer_id(name: str, num_layers: int) -> int:
    m = _LAYER.search(name)
    if m:
        return int(m.group(1)) + 1
    if "embedding" in name or "embed_tokens" in name or "wte" in name:
        return 0
    return num_layers + 1


def get_optimizer_grouped_parameters(model: Optional[torch.nn.Module] = None, weight_decay: float = 0.0,
                                     dynamic_lr_schedule=None, layer_scale: bool = False,
                                     layer_decay: float = 1.0) -> List[Dict]:
    """``[{"params": [...], "weight_decay": wd, "lr_scale": s, "name": ...}, ...]`` over the trainable parameters."""
    if model is None:
        raise ValueError("a model is required")
    skip = set(model.no_weight_decay()) if hasattr(model, "no_weight_decay") else set()
    keywords = tuple(model.no_weight_decay_keywords()) if hasattr(model, "no_weight_decay_keywords") else ()
    named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
    layer_ids = [int(m.group(1)) for n, _ in named for m in [_LAYER.search(n)] if m]
    num_layers = (max(layer_ids) + 1) if layer_ids else 0
    if dynamic_lr_schedule is not None and layer_scale:
        logger.warning("layer_scale cannot be combined with a dynamic lr schedule object per group: layer_scale is ignored")
        layer_scale = False
    groups: Dict[str, Dict] = {}
    for name, p in named:
        no_decay = p.dim() <= 1 or name.endswith(".bias") or name in skip or any(k in name for k in keywords) \
            or getattr(p, "no_weight_decay", False)
        key = "no_decay" if no_decay else "decay"
        scale = 1.0
        if layer_scale:
            lid = _layer_id(name, num_layers)
            key = f"layer_{lid}_{key}"
            scale = float(layer_decay) ** (num_layers + 1 - lid)
        g = groups.setdefault(key, {"params": [], "weight_decay": 0.0 if no_decay else float(weight_decay),
                                    "lr_scale": scale, "name": key})
        g["params"].append(p)
    return list(groups.values())
