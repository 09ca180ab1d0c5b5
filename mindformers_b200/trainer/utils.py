"""Checkpoint loading and resume bookkeeping of the trainers.

Reference: ``mindformers/trainer/utils.py`` — ``load_resume_context_from_checkpoint`` (:303-375: epoch, step, loss
scale and global batch size out of the checkpoint; the step count is rescaled when the global batch size changed),
``transform_and_load_checkpoint`` (:386-456: with ``auto_trans_ckpt`` a checkpoint written under another parallel
layout is merged with its strategy files and re-sliced for the current one before loading) and ``load_ckpt``.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist

from ..checkpoint.io import load_checkpoint
from ..checkpoint.resume import get_resume_checkpoint, rescale_resume_step
from ..tools.logger import logger


def _barrier():
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.barrier()


def _rank() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def load_resume_context_from_checkpoint(scalars: dict, path: str, resume_training, global_batch_size: int,
                                        steps_per_epoch: int) -> dict:
    """Where training continues, from the scalar entries of the loaded checkpoint (falling back to the resume point of
    the directory): ``{"initial_epoch", "initial_step", "global_step", "loss_scale", "global_batch_size"}``.
    ``initial_epoch`` counts finished epochs, ``initial_step`` the steps done inside the current one."""
    point = get_resume_checkpoint(path, resume_training) if os.path.isdir(path) else None
    epoch = int(scalars.get("epoch_num", point[0] if point else 1))
    step = int(scalars.get("step_num", point[1] if point else 0))
    old_gbs = scalars.get("global_batch_size")
    step = rescale_resume_step(step, old_gbs, global_batch_size)
    start_epoch, start_step = max(epoch - 1, 0), step
    if steps_per_epoch and start_step >= steps_per_epoch:
        start_epoch, start_step = start_epoch + start_step // steps_per_epoch, start_step % steps_per_epoch
    if old_gbs and int(old_gbs) != int(global_batch_size):
        logger.info("global batch size changed %s -> %s: resume step rescaled to %d", old_gbs, global_batch_size, step)
    return {"initial_epoch": start_epoch, "initial_step": start_step,
            "global_step": int(scalars.get("global_step", start_epoch * (steps_per_epoch or 0) + start_step)),
            "loss_scale": scalars.get("loss_scale"), "global_batch_size": global_batch_size}


def transform_checkpoint_if_needed(config, path: str) -> str:
    """With ``auto_trans_ckpt`` and a ``rank_N`` checkpoint whose strategy files are given
    (``src_strategy_path_or_dir``), merge it into one full checkpoint under ``<output_dir>/transformed_checkpoint``
    (rank 0 writes, everyone waits) and return that directory; otherwise return ``path``. Loading a full checkpoint
    slices every tensor for the current layout, so the pair merge + load is the resharding."""
    if not config.get("auto_trans_ckpt") or not os.path.isdir(path):
        return path
    if not any(d.startswith("rank_") for d in os.listdir(path)):
        return path                                      # already a full (or Hugging Face) checkpoint
    strategy = config.get("src_strategy_path_or_dir")
    if not strategy:
        guess = os.path.join(os.path.dirname(os.path.normpath(path)), "strategy")
        strategy = guess if os.path.isdir(guess) else None
    if not strategy or not os.path.isdir(strategy):
        raise ValueError("auto_trans_ckpt needs src_strategy_path_or_dir: the directory with the "
                         "ckpt_strategy_rank_N.json files of the run that wrote the checkpoint")
    dst = os.path.join(config.get("output_dir") or "./output", "transformed_checkpoint")
    point = get_resume_checkpoint(path, config.get("resume_training") or True)
    if _rank() == 0:
        from ..checkpoint.transform import unify_checkpoints
        unify_checkpoints(path, strategy, dst, include_optimizer=bool(config.get("resume_training")), point=point)
        logger.info("checkpoint %s merged into %s for the current parallel layout", path, dst)
    _barrier()
    return dst


def common_resume_point(config, path: str):
    """(epoch, step) that every rank loads from a ``rank_N`` checkpoint directory: the newest save that all rank
    directories hold and that is not marked unhealthy (or the save a file name in ``resume_training`` names). Rank 0
    records it under ``<output>/resume_record`` and all ranks read that record, so they cannot disagree. ``None`` for
    paths that are not ``rank_N`` layouts."""
    if not os.path.isdir(path) or not any(d.startswith("rank_") for d in os.listdir(path)):
        return None
    from ..checkpoint.resume import record_resume_point
    point = get_resume_checkpoint(path, config.get("resume_training") or True)
    if point is None:
        raise FileNotFoundError(f"no checkpoint under {path} is present (and healthy) in every rank directory")
    return record_resume_point(config.get("output_dir") or "./output", *point)


def load_ckpt(config, model: torch.nn.Module, optimizer=None, path: Optional[str] = None, strict: bool = False,
              family: str = "llama") -> dict:
    """Load weights (and optimizer state when given) from ``path`` or ``config.load_checkpoint``; returns the scalar
    entries of the checkpoint. From a ``rank_N`` directory every rank takes the file of the common resume point."""
    path = path or config.get("load_checkpoint")
    if not path:
        return {}
    point = common_resume_point(config, path)
    return load_checkpoint(model, path, optimizer=optimizer, strict=strict, family=family, point=point)


def transform_and_load_checkpoint(config, model: torch.nn.Module, optimizer=None, path: Optional[str] = None,
                                  family: str = "llama", resume: bool = False) -> dict:
    """``transform_checkpoint_if_needed`` + ``load_ckpt``. With ``resume`` the optimizer state and the scalars are
    restored and missing parameters are an error; otherwise only the weights are taken."""
    path = path or config.get("load_checkpoint")
    if not path:
        return {}
    path = transform_checkpoint_if_needed(config, path)
    if resume:
        return load_ckpt(config, model, optimizer, path, strict=True, family=family)
    scalars = load_ckpt(config, model, None, path, strict=False, family=family)
    if optimizer is not None and hasattr(optimizer, "reload_model_params"):
        optimizer.reload_model_params()
    return scalars
