"""Pick a consistent resume point across ranks and restore the training position.

Follows the reference's ``tools/resume_ckpt.py`` (:45-157,188-275) and ``trainer/utils.py:303-375``: every rank
directory carries a ``meta.json``; the resume point is the minimum (epoch, step) over ranks for which every rank
has a file; rank 0 records it in ``resume_record/latest_checkpointed_iteration.txt``; checkpoints listed as
unhealthy in ``health_ckpts.json`` are skipped; the step count is rescaled when the global batch size changed.
"""
from __future__ import annotations

import json
import os
from typing import List, Optional, Tuple

from ..tools.logger import logger
from ..tools.utils import barrier_world, get_real_rank, parse_ckpt_name


def _rank_dirs(directory: str) -> List[str]:
    if not os.path.isdir(directory):
        return []
    return sorted((d for d in os.listdir(directory) if d.startswith("rank_") and
                   os.path.isdir(os.path.join(directory, d))), key=lambda d: int(d.split("_")[1]))


def _available(rank_dir: str) -> List[Tuple[int, int, str]]:
    out = []
    for f in os.listdir(rank_dir):
        parsed = parse_ckpt_name(f)
        if parsed and f.endswith(".safetensors"):
            out.append((parsed[2], parsed[3], f))
    return sorted(out)


def _unhealthy(directory: str) -> set:
    path = os.path.join(directory, "health_ckpts.json")
    if not os.path.exists(path):
        return set()
    try:
        with open(path) as f:
            data = json.load(f)
    except (OSError, ValueError):
        return set()
    return {(e["epoch"], e["step"]) for e in data.get("unhealthy", [])}


def get_resume_checkpoint(directory: str, resume_training=True, expected_ranks: Optional[int] = None) -> Optional[Tuple[int, int]]:
    """(epoch, step) of the newest checkpoint that every rank directory contains, or None.

    ``resume_training`` may name a file (``prefix_rank_0-3_200.safetensors``): its epoch/step are used.
    """
    if isinstance(resume_training, str):
        parsed = parse_ckpt_name(resume_training)
        if parsed is None:
            raise ValueError(f"{resume_training!r} is not a checkpoint file name")
        return parsed[2], parsed[3]
    ranks = _rank_dirs(directory)
    if not ranks or (expected_ranks and len(ranks) < expected_ranks):
        return None
    bad = _unhealthy(directory)
    common = None
    for r in ranks:
        have = {(e, s) for e, s, _ in _available(os.path.join(directory, r))} - bad
        common = have if common is None else (common & have)
    if not common:
        return None
    # do not go past the oldest "last saved" position recorded in the meta files
    limit = None
    for r in ranks:
        meta = os.path.join(directory, r, "meta.json")
        if os.path.exists(meta):
            try:
                with open(meta) as f:
                    m = json.load(f)
                pos = (m["last_epoch"], m["last_step"])
                limit = pos if limit is None else min(limit, pos)
            except (OSError, ValueError, KeyError):
                logger.warning("unreadable %s is ignored", meta)
    ok = [c for c in common if limit is None or c <= limit]
    return max(ok) if ok else None


def record_resume_point(output_root: str, epoch: int, step: int):
    """Rank 0 writes the chosen point, all ranks synchronise, then everyone can read it."""
    d = os.path.join(output_root, "resume_record")
    if get_real_rank() == 0:
        os.makedirs(d, exist_ok=True)
        tmp = os.path.join(d, "latest_checkpointed_iteration.txt.tmp")
        with open(tmp, "w") as f:
            f.write(f"{epoch}_{step}")
        os.replace(tmp, os.path.join(d, "latest_checkpointed_iteration.txt"))
    barrier_world("resume record")
    with open(os.path.join(d, "latest_checkpointed_iteration.txt")) as f:
        e, s = f.read().strip().split("_")
    return int(e), int(s)


def checkpoint_file_for(directory: str, rank: int, epoch: int, step: int) -> Optional[str]:
    rd = os.path.join(directory, f"rank_{rank}")
    if not os.path.isdir(rd):
        return None
    for e, s, f in _available(rd):
        if (e, s) == (epoch, step):
            return os.path.join(rd, f)
    return None


def rescale_resume_step(step: int, old_global_batch: Optional[int], new_global_batch: int) -> int:
    """Keep the number of consumed samples when the global batch size changed between runs."""
    if not old_global_batch or old_global_batch == new_global_batch:
        return step
    return int(step * old_global_batch / new_global_batch)


def mark_unhealthy(directory: str, epoch: int, step: int, reason: str = ""):
    path = os.path.join(directory, "health_ckpts.json")
    data = {"unhealthy": []}
    if os.path.exists(path):
        try:
            with open(path) as f:
                data = json.load(f)
        except (OSError, ValueError):
            pass
    data.setdefault("unhealthy", []).append({"epoch": epoch, "step": step, "reason": reason})
    tmp = path + ".tmp"
    with open(tmp, "w") as f:
        json.dump(data, f)
    os.replace(tmp, path)
