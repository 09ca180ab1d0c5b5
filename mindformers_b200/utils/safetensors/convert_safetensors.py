"""Hugging Face safetensors directory → framework names and fused layouts, several processes at a time.

The reference converts large checkpoints with a pool of processes, one input file each, concatenating q / k / v and
gate / up on the way (``utils/safetensors/convert_safetensors.py:27-119``). The fused layouts need all tensors of a
layer together and HF shards may cut a layer in two, so here the unit of work is a LAYER, not a file: the parent
indexes which file holds which tensor, every worker opens the files it needs with ``safe_open`` (memory-mapped, only
the requested tensors are read), converts its layers and writes one output file; the parent writes the
``model.safetensors.index.json`` that makes the directory loadable like any sharded checkpoint.
"""
from __future__ import annotations

import json
import multiprocessing as mp
import os
import re
from typing import Dict, List, Optional

_LAYER = re.compile(r"(?:^|\.)layers\.(\d+)\.")


def _index_keys(src_dir: str) -> Dict[str, str]:
    from safetensors import safe_open
    idx_file = os.path.join(src_dir, "model.safetensors.index.json")
    if os.path.exists(idx_file):
        with open(idx_file) as f:
            return dict(json.load(f)["weight_map"])
    out = {}
    for fn in sorted(os.listdir(src_dir)):
        if fn.endswith(".safetensors"):
            with safe_open(os.path.join(src_dir, fn), framework="pt") as f:
                for k in f.keys():
                    out[k] = fn
    return out


def _convert_group(job):
    src_dir, dst_dir, part, keys_by_file, cfg_dict, family, dtype_name, keep_fp8 = job
    import torch
    from safetensors import safe_open
    from safetensors.torch import save_file
    from ...checkpoint import name_maps
    from ...models.presets import preset_is_mla
    from ...parallel.transformer_config_utils import convert_to_transformer_config
    torch.set_num_threads(1)
    sd = {}
    for fn, keys in keys_by_file.items():
        with safe_open(os.path.join(src_dir, fn), framework="pt") as f:
            for k in keys:
                sd[k] = f.get_tensor(k)
    cfg = convert_to_transformer_config(dict(cfg_dict), is_mla_model=preset_is_mla(cfg_dict), strict=False)
    dtype = getattr(torch, dtype_name) if dtype_name else None
    out = name_maps.hf_to_framework(sd, cfg, family, dtype, keep_fp8=keep_fp8)
    out = {k: v.contiguous() for k, v in out.items()}
    name = f"model-{part:05d}.safetensors"
    save_file(out, os.path.join(dst_dir, name), metadata={"format": "pt"})
    return name, {k: int(v.numel() * v.element_size()) for k, v in out.items()}


def convert_hf_safetensors_multiprocess(src_dir: str, dst_dir: str, config: dict, family: str = "llama",
                                        dtype: Optional[str] = None, workers: int = 4, keep_fp8: bool = False,
                                        layers_per_file: Optional[int] = None) -> str:
    """Convert ``src_dir`` (HF names) into ``dst_dir`` (framework names, fused QKV / gate-up / expert stacks) with
    ``workers`` processes. ``config``: the model's ``config.json`` mapping. Returns the path of the index file."""
    key_file = _index_keys(src_dir)
    if not key_file:
        raise FileNotFoundError(f"no safetensors files in {src_dir}")
    os.makedirs(dst_dir, exist_ok=True)
    groups: Dict[int, List[str]] = {}
    for k in key_file:
        m = _LAYER.search(k)
        groups.setdefault(int(m.group(1)) if m else -1, []).append(k)
    layer_ids = sorted(g for g in groups if g >= 0)
    per = layers_per_file or max(1, -(-len(layer_ids) // max(1, workers * 2)))
    units: List[List[str]] = []
    if -1 in groups:
        units.append(groups[-1])                          # embeddings, final norm, head, anything outside the layers
    for i in range(0, len(layer_ids), per):
        units.append([k for lid in layer_ids[i:i + per] for k in groups[lid]])
    jobs = []
    for part, keys in enumerate(units):
        by_file: Dict[str, List[str]] = {}
        for k in keys:
            by_file.setdefault(key_file[k], []).append(k)
        jobs.append((src_dir, dst_dir, part, by_file, dict(config), family, dtype, keep_fp8))
    if workers <= 1 or len(jobs) == 1:
        results = [_convert_group(j) for j in jobs]
    else:
        with mp.get_context("spawn").Pool(min(workers, len(jobs))) as pool:
            results = pool.map(_convert_group, jobs)
    weight_map, total = {}, 0
    for name, sizes in results:
        for k, n in sizes.items():
            if k in weight_map:
                raise RuntimeError(f"{k} was produced by two conversion units")
            weight_map[k] = name
            total += n
    index = os.path.join(dst_dir, "model.safetensors.index.json")
    with open(index, "w") as f:
        json.dump({"metadata": {"total_size": total, "format": "framework"}, "weight_map": weight_map}, f, indent=1)
    return index
