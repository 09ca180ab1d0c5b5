"""Small helpers: ranks, output directories, checkpoint file names, barriers, pipeline-stage bookkeeping.

Counterpart of the reference's ``tools/utils.py`` (``set_output_path`` :160, ``get_output_subpath`` :190,
``get_real_rank`` :454, ``get_real_group_size`` :479, ckpt-name parsing :627-680, ``barrier_world`` :730,
``get_pipeline_rank_ids`` :742, ``calculate_pipeline_stage`` :773).
"""
from __future__ import annotations

import os
import re
from typing import List, Optional, Tuple

import torch.distributed as dist

_OUTPUT_ROOT = "./output"
PARALLEL_SUBDIRS = ("checkpoint", "checkpoint_network", "checkpoint_trainable", "strategy", "log", "profile",
                    "resume_record", "unified_checkpoint", "merged_strategy", "ms_safetensors")


def get_real_rank() -> int:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank()
    return int(os.environ.get("RANK", os.environ.get("RANK_ID", "0")))


def get_real_group_size() -> int:
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size()
    return int(os.environ.get("WORLD_SIZE", os.environ.get("RANK_SIZE", "1")))


def is_main_rank() -> bool:
    return get_real_rank() == 0


def set_output_path(path: Optional[str]):
    global _OUTPUT_ROOT
    _OUTPUT_ROOT = os.path.expanduser(path or "./output")
    os.environ["LOCAL_DEFAULT_PATH"] = _OUTPUT_ROOT
    os.makedirs(_OUTPUT_ROOT, exist_ok=True)
    return _OUTPUT_ROOT


def get_output_root_path() -> str:
    return os.environ.get("LOCAL_DEFAULT_PATH", _OUTPUT_ROOT)


def get_output_subpath(sub_class: str, rank_id: Optional[int] = None, append_rank: bool = True) -> str:
    """``<output>/<sub_class>[/rank_<r>]`` (created on demand)."""
    if not isinstance(sub_class, str) or not sub_class:
        raise ValueError("sub_class must be a non-empty string")
    root = os.path.join(get_output_root_path(), sub_class.strip("/"))
    if append_rank:
        root = os.path.join(root, f"rank_{get_real_rank() if rank_id is None else rank_id}")
    os.makedirs(root, exist_ok=True)
    return root


def barrier_world(action: Optional[str] = None):
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()


_CKPT_RE = re.compile(r"^(?P<prefix>.+?)(?:_rank_(?P<rank>\d+))?-(?P<epoch>\d+)_(?P<step>\d+)\.(?P<ext>ckpt|safetensors)$")


def parse_ckpt_name(filename: str) -> Optional[Tuple[str, int, int, int]]:
    """``prefix_rank_3-2_100.safetensors`` → ``(prefix, 3, 2, 100)``; ``None`` when the name does not match."""
    m = _CKPT_RE.match(os.path.basename(filename))
    if not m:
        return None
    return m["prefix"], int(m["rank"] or 0), int(m["epoch"]), int(m["step"])


def format_ckpt_name(prefix: str, rank: int, epoch: int, step: int, ext: str = "safetensors") -> str:
    return f"{prefix}_rank_{rank}-{epoch}_{step}.{ext}"


def get_epoch_and_step_from_ckpt_name(filename: str) -> Tuple[int, int]:
    parsed = parse_ckpt_name(filename)
    if parsed is None:
        raise ValueError(f"{filename!r} does not look like '<prefix>_rank_<r>-<epoch>_<step>.<ext>'")
    return parsed[2], parsed[3]


def get_last_checkpoint(directory: str, ext: str = "safetensors") -> Optional[str]:
    """Newest checkpoint file of a rank directory by (epoch, step)."""
    best = None
    if not os.path.isdir(directory):
        return None
    for f in os.listdir(directory):
        parsed = parse_ckpt_name(f)
        if parsed and f.endswith("." + ext):
            key = (parsed[2], parsed[3])
            if best is None or key > best[0]:
                best = (key, os.path.join(directory, f))
    return best[1] if best else None


def calculate_pipeline_stage(layers_per_stage: List[int], model_layers: List[int], input_layers_name=None) -> List[int]:
    """Stage index of every layer given the number of layers on each stage."""
    out = []
    for stage, n in enumerate(layers_per_stage):
        out += [stage] * n
    if len(out) != sum(model_layers):
        raise ValueError("layers_per_stage does not add up to the number of layers")
    return out


def get_pipeline_rank_ids() -> List[int]:
    """One rank of every pipeline stage (the first rank of the stage), used to pick profiling ranks."""
    from ..parallel import parallel_state as ps
    pp = ps.get_pipeline_model_parallel_world_size()
    world = get_real_group_size()
    per = max(1, world // pp)
    return [s * per for s in range(pp)]


def str2bool(v) -> bool:
    if isinstance(v, bool):
        return v
    if str(v).lower() in ("true", "1", "yes", "y"):
        return True
    if str(v).lower() in ("false", "0", "no", "n"):
        return False
    raise ValueError(f"cannot interpret {v!r} as a boolean")
