"""Offline resharding: merge per-rank checkpoints into full tensors, and re-slice for another layout.

Plays the role of the reference's ``toolkit/safetensors/unified_safetensors.py`` and
``tools/ckpt_transform/transform_checkpoint.py`` (``TransformCkpt`` :57-360) using the JSON strategy files
written next to the checkpoints instead of MindSpore strategy protobufs.

    python -m mindformers_b200.checkpoint.transform --src output/checkpoint --strategy output/strategy --dst unified
"""
from __future__ import annotations

import argparse
import glob
import json
import os
from typing import Dict, List

import torch
from safetensors.torch import load_file, save_file

from ..tools.utils import parse_ckpt_name
from .sharding import merge_shards


def _latest(rank_dir: str) -> str:
    files = [f for f in glob.glob(os.path.join(rank_dir, "*.safetensors")) if parse_ckpt_name(f)]
    if not files:
        raise FileNotFoundError(f"no checkpoint in {rank_dir}")
    return max(files, key=lambda f: parse_ckpt_name(f)[2:])


def unify_checkpoints(src_dir: str, strategy_dir: str, dst_dir: str, include_optimizer: bool = True) -> str:
    """Merge the newest checkpoint of every ``rank_N`` directory into one full checkpoint.

    Ranks are combined by their tensor-parallel position (same-position data-parallel replicas are identical;
    the first one is used). Optimizer moments follow their parameter; scalars go to ``hyper_param.safetensors``.
    """
    ranks = sorted((d for d in os.listdir(src_dir) if d.startswith("rank_")), key=lambda d: int(d.split("_")[1]))
    strategies = {}
    for d in ranks:
        r = int(d.split("_")[1])
        with open(os.path.join(strategy_dir, f"ckpt_strategy_rank_{r}.json")) as f:
            strategies[r] = json.load(f)
    shards: Dict[str, Dict[int, torch.Tensor]] = {}
    layouts: Dict[str, dict] = {}
    scalars: Dict[str, torch.Tensor] = {}
    for d in ranks:
        r = int(d.split("_")[1])
        sd = load_file(_latest(os.path.join(src_dir, d)))
        params = strategies[r]["params"]
        for name, t in sd.items():
            base = name
            for pre in ("adam_m.", "adam_v.", "master_lo."):
                if name.startswith(pre):
                    base = name[len(pre):]
            if base in params:
                if name != base and not include_optimizer:
                    continue
                lay = params[base]
                pos = lay.get("tp_rank", 0) + lay.get("tp", 1) * lay.get("ep_rank", 0)
                shards.setdefault(name, {}).setdefault(pos, t)
                layouts[name] = lay
            elif name.startswith("__shard__"):
                continue
            elif t.dim() == 0:
                scalars.setdefault(name, t)
    full: Dict[str, torch.Tensor] = {}
    for name, by_pos in shards.items():
        lay = layouts[name]
        tp, ep = lay.get("tp", 1), lay.get("ep", 1)
        per_ep = []
        for e in range(ep):
            tps = [by_pos[p + tp * e] for p in range(tp) if (p + tp * e) in by_pos]
            if len(tps) != tp:
                raise ValueError(f"shards of {name} are incomplete: have positions {sorted(by_pos)}")
            per_ep.append(merge_shards(tps, lay))
        full[name] = torch.cat(per_ep, dim=0) if ep > 1 else per_ep[0]
    os.makedirs(dst_dir, exist_ok=True)
    save_file({k: v.contiguous() for k, v in full.items() if not k.startswith(("adam_", "master_lo."))},
              os.path.join(dst_dir, "model.safetensors"), metadata={"format": "pt"})
    hyper = {k: v.contiguous() for k, v in full.items() if k.startswith(("adam_", "master_lo."))}
    hyper.update(scalars)
    if hyper:
        save_file(hyper, os.path.join(dst_dir, "hyper_param.safetensors"), metadata={"format": "pt"})
    return dst_dir


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--src", required=True, help="directory with rank_N sub-directories")
    ap.add_argument("--strategy", required=True, help="directory with ckpt_strategy_rank_N.json files")
    ap.add_argument("--dst", required=True)
    ap.add_argument("--no-optimizer", action="store_true")
    args = ap.parse_args(argv)
    print(unify_checkpoints(args.src, args.strategy, args.dst, include_optimizer=not args.no_optimizer))


if __name__ == "__main__":
    main()
