"""Checkpoint loading helpers under the reference's path (``utils/load_checkpoint_utils.py``)."""
from ..checkpoint.io import is_hf_safetensors_dir, load_checkpoint, resolve_checkpoint  # noqa: F401
from ..trainer.utils import load_ckpt, transform_and_load_checkpoint  # noqa: F401
from ..checkpoint.transform import unify_checkpoints  # noqa: F401

__all__ = ["is_hf_safetensors_dir", "load_checkpoint", "load_ckpt", "resolve_checkpoint", "transform_and_load_checkpoint", "unify_checkpoints"]
