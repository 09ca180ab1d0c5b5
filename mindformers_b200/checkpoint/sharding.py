"""Slice full tensors into the shards a rank owns, and merge shards back.

A parameter describes its own layout through attributes set by the parallel layers: ``tensor_model_parallel``,
``partition_dim``, ``partition_sections`` (e.g. q|k|v or gate|up, each sharded separately), ``is_expert``
(expert-parallel slice of dim 0). The same description is written next to rank checkpoints as a JSON "strategy"
file, which replaces the MindSpore strategy protobufs the reference uses for resharding
(``utils/load_checkpoint_utils.py:222-236,507-549``).
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional

import torch

from ..parallel import parallel_state as ps
from ..parallel.layers.tensor_parallel import shard_sections


def param_layout(name: str, p: torch.Tensor) -> dict:
    tp = ps.get_tensor_model_parallel_world_size()
    ep = ps.get_expert_model_parallel_world_size()
    lay = {"shape": list(p.shape), "tp": 1, "dim": -1, "sections": None, "ep": 1}
    if getattr(p, "is_expert", False) and ep > 1:
        lay.update(ep=ep, ep_rank=ps.get_expert_model_parallel_rank())
    if getattr(p, "tensor_model_parallel", False) and tp > 1:
        lay.update(tp=tp, dim=int(getattr(p, "partition_dim", 0)), tp_rank=ps.get_tensor_model_parallel_rank(),
                   sections=list(getattr(p, "partition_sections", None) or []) or None,
                   groups=list(getattr(p, "partition_groups", None) or []) or None)
    return lay


def shard_for_param(full: torch.Tensor, p: torch.Tensor) -> torch.Tensor:
    """The slice of ``full`` that parameter ``p`` of this rank holds."""
    lay = param_layout("", p)
    t = full
    if lay["ep"] > 1:
        per = t.shape[0] // lay["ep"]
        t = t[lay["ep_rank"] * per:(lay["ep_rank"] + 1) * per]
    if lay["tp"] > 1:
        dim, rank, tp = lay["dim"], lay["tp_rank"], lay["tp"]
        if lay["sections"]:
            t = shard_sections(t, lay["sections"], dim, rank, tp, lay.get("groups"))
        else:
            n = t.shape[dim]
            per = p.shape[dim]
            if per * tp != n:  # padded vocabulary: pad the full tensor first
                pad = per * tp - n
                shape = list(t.shape)
                shape[dim] = pad
                t = torch.cat((t, t.new_zeros(shape)), dim=dim)
            t = t.narrow(dim, rank * per, per)
    if tuple(t.shape) != tuple(p.shape):
        raise ValueError(f"checkpoint tensor of shape {tuple(full.shape)} does not fit parameter {tuple(p.shape)}")
    return t.contiguous()


def model_strategy(model: torch.nn.Module) -> Dict[str, dict]:
    return {n: param_layout(n, p) for n, p in model.named_parameters()}


def save_strategy(model: torch.nn.Module, path: str):
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    info = {"tp": ps.get_tensor_model_parallel_world_size(), "pp": ps.get_pipeline_model_parallel_world_size(),
            "ep": ps.get_expert_model_parallel_world_size(), "params": model_strategy(model)}
    with open(path, "w") as f:
        json.dump(info, f)


def merge_shards(shards: List[torch.Tensor], layout: dict, full_rows: Optional[int] = None) -> torch.Tensor:
    """Inverse of the tensor-parallel slicing for one parameter (``shards`` ordered by tp rank)."""
    tp, dim, sections = layout.get("tp", 1), layout.get("dim", -1), layout.get("sections")
    if tp <= 1 or dim < 0:
        return shards[0]
    if sections:
        groups = layout.get("groups")
        from ..parallel.layers.tensor_parallel import section_local_sizes
        per = section_local_sizes(sections, tp, groups)
        pieces = [torch.split(s, per, dim=dim) for s in shards]
        out = []
        for i in range(len(sections)):
            g = groups[i] if groups else None
            # a replicated section: one copy of each group, taken from the first rank that holds it
            ranks = [j * tp // g for j in range(g)] if g and g < tp else range(tp)
            out.append(torch.cat([pieces[r][i] for r in ranks], dim=dim))
        return torch.cat(out, dim=dim)
    out = torch.cat(shards, dim=dim)
    if full_rows is not None and out.shape[dim] > full_rows:
        out = out.narrow(dim, 0, full_rows)
    return out
