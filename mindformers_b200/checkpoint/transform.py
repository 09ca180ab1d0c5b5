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


_STATE_PREFIXES = ("adam_m.", "adam_v.", "master_lo.")


def unify_checkpoints(src_dir: str, strategy_dir: str, dst_dir: str, include_optimizer: bool = True,
                      point=None) -> str:
    """Merge one save of every ``rank_N`` directory into one full checkpoint.

    The save is ``point`` = (epoch, step) when given, else the newest one that EVERY rank directory holds (ranks
    can differ by one save after a crash). Ranks are combined by their tensor- / expert-parallel position;
    data-parallel replicas of a parameter are identical and the first one is used. Optimizer states follow their
    parameter: under a sharded optimizer each data-parallel rank wrote a flat slice of the local tensor with its
    ``__slice__.<param>`` = [offset, count, numel]; the slices of one position are stitched back together before
    the tensor-parallel merge, and a hole raises. Pipeline stages hold disjoint parameters under global layer
    numbers, so they simply add up. Scalars go to ``hyper_param.safetensors`` with the optimizer states.
    """
    from .resume import checkpoint_file_for, get_resume_checkpoint
    ranks = sorted((d for d in os.listdir(src_dir) if d.startswith("rank_")), key=lambda d: int(d.split("_")[1]))
    if point is None:
        point = get_resume_checkpoint(src_dir, True)
    strategies = {}
    for d in ranks:
        r = int(d.split("_")[1])
        with open(os.path.join(strategy_dir, f"ckpt_strategy_rank_{r}.json")) as f:
            strategies[r] = json.load(f)
    shards: Dict[str, Dict[int, torch.Tensor]] = {}
    pieces: Dict[str, Dict[int, list]] = {}          # sliced optimizer states: name -> position -> [(offset, flat)]
    layouts: Dict[str, dict] = {}
    scalars: Dict[str, torch.Tensor] = {}
    for d in ranks:
        r = int(d.split("_")[1])
        path = checkpoint_file_for(src_dir, r, *point) if point is not None else None
        sd = load_file(path or _latest(os.path.join(src_dir, d)))
        params = strategies[r]["params"]
        for name, t in sd.items():
            if name.startswith("__slice__."):
                continue
            base = name
            for pre in _STATE_PREFIXES:
                if name.startswith(pre):
                    base = name[len(pre):]
            if base in params:
                if name != base and not include_optimizer:
                    continue
                lay = params[base]
                pos = lay.get("tp_rank", 0) + lay.get("tp", 1) * lay.get("ep_rank", 0)
                layouts[name] = lay
                sl = sd.get(f"__slice__.{base}") if name != base else None
                if sl is not None and t.dim() == 1 and t.numel() == int(sl[1]):
                    pieces.setdefault(name, {}).setdefault(pos, []).append((int(sl[0]), t))
                else:
                    shards.setdefault(name, {}).setdefault(pos, t)
            elif t.dim() == 0:
                scalars.setdefault(name, t)
    for name, by_pos in pieces.items():
        lay = layouts[name]
        numel = 1
        for x in lay["shape"]:
            numel *= int(x)
        for pos, lst in by_pos.items():
            if pos in shards.get(name, {}):
                continue                                   # a replica held the whole tensor
            flat = torch.empty(numel, dtype=lst[0][1].dtype)
            covered = 0
            for off, t in sorted(lst, key=lambda x: x[0]):
                if off > covered:
                    raise ValueError(f"optimizer state {name}: elements [{covered}, {off}) of position {pos} are in no "
                                     "rank file (a data-parallel rank's checkpoint is missing)")
                flat[off:off + t.numel()] = t
                covered = max(covered, off + t.numel())
            if covered < numel:
                raise ValueError(f"optimizer state {name}: elements [{covered}, {numel}) of position {pos} are missing")
            shards.setdefault(name, {})[pos] = flat.view(lay["shape"])
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
    save_file({k: v.contiguous() for k, v in full.items() if not k.startswith(_STATE_PREFIXES)},
              os.path.join(dst_dir, "model.safetensors"), metadata={"format": "pt"})
    hyper = {k: v.contiguous() for k, v in full.items() if k.startswith(_STATE_PREFIXES)}
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
