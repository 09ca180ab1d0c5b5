"""Choice of the checkpoint to resume from (reference ``mindformers/tools/resume_ckpt.py``: ``get_resume_checkpoint`` :45,
``get_resume_checkpoint_by_meta`` :188, health filter :131-157). The implementation lives in ``checkpoint/resume.py``;
this module keeps the reference's import path and entry points."""
from __future__ import annotations

import os
from typing import Optional

from ..checkpoint.resume import (checkpoint_file_for, get_resume_checkpoint as _resume_point, mark_unhealthy,  # noqa: F401
                                 record_resume_point)


def get_resume_checkpoint_by_meta(checkpoint_dir: str, ckpt_format: str = "safetensors", use_checkpoint_health_monitor: bool = False,
                                  health_ckpts_record_dir: Optional[str] = None):
    """The newest (epoch, step) that every ``rank_N`` directory holds and that is not marked unhealthy, as the file name
    of rank 0's checkpoint (the reference returns the name that all ranks then derive their own from)."""
    point = _resume_point(checkpoint_dir, True)
    if point is None:
        return None
    path = checkpoint_file_for(checkpoint_dir, 0, *point)
    return os.path.basename(path) if path else None


def get_resume_checkpoint(checkpoint_dir: str, resume_training=True, resume_by_meta: bool = True, ckpt_format: str = "safetensors",
                          use_checkpoint_health_monitor: bool = False, health_ckpts_record_dir: Optional[str] = None):
    """``resume_training`` naming a file wins; otherwise the common, healthy resume point (see above)."""
    if isinstance(resume_training, str) and resume_training:
        return resume_training
    if not resume_training:
        return None
    return get_resume_checkpoint_by_meta(checkpoint_dir, ckpt_format, use_checkpoint_health_monitor, health_ckpts_record_dir)
