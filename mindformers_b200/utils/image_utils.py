"""Image layout helpers of the multimodal processors: channel-dimension bookkeeping, best-fit resolution for
"any resolution" vision towers and patch division.

API counterpart of the reference's ``utils/image_utils.py`` (``ChannelDimension`` :35, ``PaddingMode`` :43,
``infer_channel_dimension_format`` :53, ``get_image_size`` :85, ``select_best_resolution`` :108, ``divide_to_patches``
:145)."""
from __future__ import annotations

from enum import Enum
from typing import List, Optional, Sequence, Tuple, Union

import numpy as np


class ExplicitEnum(str, Enum):
    @classmethod
    def _missing_(cls, value):
        raise ValueError(f"{value!r} is not a valid {cls.__name__}; choose from {[m.value for m in cls]}")


class ChannelDimension(ExplicitEnum):
    FIRST = "channels_first"
    LAST = "channels_last"


class PaddingMode(ExplicitEnum):
    CONSTANT = "constant"
    REFLECT = "reflect"
    REPLICATE = "replicate"
    SYMMETRIC = "symmetric"


def infer_channel_dimension_format(image: np.ndarray, num_channels: Optional[Union[int, Sequence[int]]] = None) -> ChannelDimension:
    """Channel-first or channel-last, decided by which of the candidate axes has a plausible channel count (1 or 3
    unless ``num_channels`` says otherwise); an image or a batch of images."""
    counts = (1, 3) if num_channels is None else ((num_channels,) if isinstance(num_channels, int) else tuple(num_channels))
    if image.ndim == 3:
        first, last = 0, 2
    elif image.ndim == 4:
        first, last = 1, 3
    else:
        raise ValueError(f"Unsupported number of image dimensions: {image.ndim}")
    if image.shape[first] in counts and image.shape[last] not in counts:
        return ChannelDimension.FIRST
    if image.shape[last] in counts:
        return ChannelDimension.LAST
    if image.shape[first] in counts:
        return ChannelDimension.FIRST
    raise ValueError("Unable to infer channel dimension format")


def get_image_size(image: np.ndarray, channel_dim: Optional[ChannelDimension] = None) -> Tuple[int, int]:
    """``(height, width)``."""
    channel_dim = ChannelDimension(channel_dim) if channel_dim is not None else infer_channel_dimension_format(image)
    if channel_dim == ChannelDimension.FIRST:
        return int(image.shape[-2]), int(image.shape[-1])
    return int(image.shape[-3]), int(image.shape[-2])


def select_best_resolution(original_size: tuple, possible_resolutions: list) -> tuple:
    """Of the candidate ``(height, width)`` canvases, the one on which the aspect-preserving down/up-scaled image keeps
    the most of its pixels; ties go to the canvas that wastes the least area."""
    oh, ow = original_size
    best, best_eff, best_waste = None, -1, float("inf")
    for h, w in possible_resolutions:
        s = min(w / ow, h / oh)
        sw, sh = int(ow * s), int(oh * s)
        eff = min(sw * sh, ow * oh)
        waste = w * h - eff
        if eff > best_eff or (eff == best_eff and waste < best_waste):
            best, best_eff, best_waste = (h, w), eff, waste
    return best


def divide_to_patches(image: np.ndarray, patch_size: int, input_data_format=None) -> List[np.ndarray]:
    """Row-major ``patch_size`` x ``patch_size`` tiles (edge tiles are smaller when the size does not divide)."""
    fmt = ChannelDimension(input_data_format) if input_data_format is not None else infer_channel_dimension_format(image)
    h, w = get_image_size(image, fmt)
    out = []
    for top in range(0, h, patch_size):
        for left in range(0, w, patch_size):
            if fmt == ChannelDimension.LAST:
                out.append(image[top:top + patch_size, left:left + patch_size])
            else:
                out.append(image[:, top:top + patch_size, left:left + patch_size])
    return out
