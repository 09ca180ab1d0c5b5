"""Offline checkpoint transformation between parallel layouts (reference ``mindformers/tools/ckpt_transform``)."""
from .transform_checkpoint import TransformCkpt, slice_for_layout

__all__ = ["TransformCkpt", "slice_for_layout"]
