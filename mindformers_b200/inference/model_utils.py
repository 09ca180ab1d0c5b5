"""Helpers shared by the models when they serve: phase flags, fused-name conversion, weight loading, strategy files.

Reference: ``parallel_core/inference/model_utils.py`` (``InferModelMixin``: prefill / decode flagging :65-81,
``convert_net_name`` — per-projection framework names to the names of the fused network, e.g.
``linear_q|k|v -> linear_qkv``, ``experts.N.gating -> experts.weight1`` :83-114 — and ``load_weights(path)`` through
``*index.json`` / ``param_name_map.json`` :116-161) and ``parallel_core/inference/utils.py`` (``generate_state_dict`` /
``save_strategy_file`` :83-244, which record how every parameter of a stand-alone model is sharded).

No dynamic-shape declaration is needed here (nothing is traced), so that part of the mixin has no counterpart.
"""
from __future__ import annotations

import json
import os
import re
from typing import Dict

import torch

from ..checkpoint.sharding import model_strategy, save_strategy
from ..parallel import parallel_state as ps

# per-projection name -> (fused parameter, which part of it)
_NET_NAME_RULES = (
    (re.compile(r"\.self_attention\.linear_(q|k|v)\.(weight|bias)$"), r".self_attention.linear_qkv.\2"),
    (re.compile(r"\.self_attention\.linear_(q_down_proj|kv_down_proj)\.(weight)$"), r".self_attention.linear_qkv.\2"),
    (re.compile(r"\.self_attention\.linear_q_up_proj\."), ".self_attention.linear_qb."),
    (re.compile(r"\.self_attention\.linear_kv_up_proj\."), ".self_attention.linear_kvb."),
    (re.compile(r"\.self_attention\.kv_layernorm\."), ".self_attention.k_layernorm."),
    (re.compile(r"\.(mlp|shared_experts)\.gating\.(weight|bias)$"), r".\1.linear_fc1.\2"),
    (re.compile(r"\.experts\.\d+\.(gating|linear_fc1)\.weight$"), ".experts.weight1"),
    (re.compile(r"\.experts\.\d+\.linear_fc2\.weight$"), ".experts.weight2"),
    (re.compile(r"\.router\.weight\.weight$"), ".router.weight"),
)


def convert_net_name(name: str) -> str:
    """Name of the fused-network parameter that a per-projection framework name ends up in."""
    for pat, rep in _NET_NAME_RULES:
        new, n = pat.subn(rep, name)
        if n:
            return new
    return name


class InferModelMixin:
    """Mixed into the model classes: phase flag, name conversion, weight loading by directory."""

    _is_prefill = True

    def set_phase(self, is_prefill: bool):
        """The generation loop marks each forward as prefill (many tokens per sequence) or decode (one)."""
        self._is_prefill = bool(is_prefill)

    @property
    def is_prefill(self) -> bool:
        return self._is_prefill

    @staticmethod
    def convert_net_name(name: str) -> str:
        return convert_net_name(name)

    def load_weights_from_dir(self, path: str, strict: bool = False, keep_fp8: bool = False) -> dict:
        """Stream a pretrained directory into the model. ``param_name_map.json`` in the directory (checkpoint name →
        framework name) is applied first when present."""
        from .weights_utils import load_weights
        family = getattr(self, "weight_family", "llama")
        name_map = os.path.join(path, "param_name_map.json")
        if os.path.exists(name_map):
            return _load_with_name_map(self, path, name_map, strict)
        return load_weights(self, path, family=family, strict=strict, keep_fp8=keep_fp8)


def _load_with_name_map(model, path: str, name_map_file: str, strict: bool) -> dict:
    from ..checkpoint.sharding import shard_for_param
    from .weights_utils import WeightsLoader
    with open(name_map_file) as f:
        name_map: Dict[str, str] = json.load(f)
    loader = WeightsLoader(path)
    params = dict(model.named_parameters())
    used = set()
    with torch.no_grad():
        for src, dst in name_map.items():
            if dst in params and loader.has(src):
                p = params[dst]
                p.copy_(shard_for_param(loader.get(src), p).to(device=p.device, dtype=p.dtype))
                used.add(dst)
    missing = [n for n in params if n not in used]
    if missing and strict:
        raise KeyError(f"{path} lacks parameters: {missing[:8]}")
    return {"tensors": len(used), "missing": missing}


def generate_state_dict(model: torch.nn.Module) -> dict:
    """``{"total_rank", "stage_rank_size", "stage", "model": {name: {shape, shard}}}``: every parameter with its local
    shape and how many ways each dimension is split (1 = replicated)."""
    out = {}
    for name, layout in model_strategy(model).items():
        shard = [1] * len(layout["shape"])
        if layout["tp"] > 1 and 0 <= layout["dim"] < len(shard):
            shard[layout["dim"]] = layout["tp"]
        if layout["ep"] > 1 and shard:
            shard[0] = layout["ep"]                     # expert stacks are split along the expert axis
        out[name] = {"shape": layout["shape"], "shard": shard}
    world = torch.distributed.get_world_size() if torch.distributed.is_available() and torch.distributed.is_initialized() else 1
    pp = ps.get_pipeline_model_parallel_world_size()
    return {"total_rank": world, "stage_rank_size": world // max(pp, 1), "stage": ps.get_pipeline_model_parallel_rank(),
            "model": out}


def save_strategy_file(model_or_state: object, path: str) -> str:
    """Write the sharding strategy of a model (or the dict of ``generate_state_dict``) as JSON; the resharding tools
    (``checkpoint/transform.py``) read it as the source or target layout."""
    if isinstance(model_or_state, torch.nn.Module):
        save_strategy(model_or_state, path)
        return path
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    with open(path, "w") as f:
        json.dump(model_or_state, f)
    return path
