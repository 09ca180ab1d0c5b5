"""Array-level image operations used by the image processors: layout conversion, rescale, normalise, resize,
centre crop and padding.

API counterpart of the reference's ``utils/image_transforms.py`` (``to_pil_image`` :56, ``to_channel_dimension_format``
:103, ``get_channel_dimension_axis`` :142, ``rescale`` :166, ``center_crop`` :204, ``normalize`` :303, ``resize`` :363,
``get_resize_output_image_size`` :430, ``pad`` :496). Images are numpy arrays; the layout is inferred unless given."""
from __future__ import annotations

from typing import Iterable, Optional, Sequence, Tuple, Union

import numpy as np
from PIL import Image

from .image_utils import ChannelDimension, PaddingMode, get_image_size, infer_channel_dimension_format

_RESAMPLE = {0: Image.NEAREST, 1: Image.LANCZOS, 2: Image.BILINEAR, 3: Image.BICUBIC, 4: Image.BOX, 5: Image.HAMMING}


def get_channel_dimension_axis(image: np.ndarray, input_data_format=None) -> int:
    fmt = ChannelDimension(input_data_format) if input_data_format is not None else infer_channel_dimension_format(image)
    return image.ndim - 3 if fmt == ChannelDimension.FIRST else image.ndim - 1


def to_channel_dimension_format(image: np.ndarray, channel_dim, input_channel_dim=None) -> np.ndarray:
    src = ChannelDimension(input_channel_dim) if input_channel_dim is not None else infer_channel_dimension_format(image)
    dst = ChannelDimension(channel_dim)
    if src == dst:
        return image
    if dst == ChannelDimension.FIRST:
        return np.moveaxis(image, -1, -3)
    return np.moveaxis(image, -3, -1)


def rescale(image: np.ndarray, scale: float, data_format=None, dtype=np.float32, input_data_format=None) -> np.ndarray:
    out = (image.astype(np.float64) * scale).astype(dtype)
    if data_format is not None:
        out = to_channel_dimension_format(out, data_format, input_data_format)
    return out


def _needs_rescale(image: np.ndarray) -> bool:
    if image.dtype == np.uint8:
        return False
    if np.allclose(image, image.astype(int)):
        if np.all(image >= 0) and np.all(image <= 255):
            return False
        raise ValueError("integer-valued image outside [0, 255]")
    if np.all(image >= 0) and np.all(image <= 1):
        return True
    raise ValueError("float image outside [0, 1]")


def to_pil_image(image, do_rescale: Optional[bool] = None, input_data_format=None) -> Image.Image:
    if isinstance(image, Image.Image):
        return image
    arr = np.asarray(image)
    arr = to_channel_dimension_format(arr, ChannelDimension.LAST, input_data_format)
    if arr.shape[-1] == 1:
        arr = arr[..., 0]
    if _needs_rescale(arr) if do_rescale is None else do_rescale:
        arr = arr * 255.0
    return Image.fromarray(np.clip(np.rint(arr), 0, 255).astype(np.uint8) if arr.dtype != np.uint8 else arr)


def get_resize_output_image_size(input_image, size: Union[int, Tuple[int, int], Sequence[int]], default_to_square: bool = True,
                                 max_size: Optional[int] = None, input_data_format=None) -> Tuple[int, int]:
    """``(height, width)`` for a requested ``size``: a pair is taken as is; an int is the square side, or with
    ``default_to_square=False`` the shorter side (aspect kept, the longer side capped at ``max_size``)."""
    if isinstance(size, (tuple, list)):
        if len(size) == 2:
            return int(size[0]), int(size[1])
        if len(size) == 1:
            size = size[0]
        else:
            raise ValueError("size must have 1 or 2 values")
    if default_to_square:
        return int(size), int(size)
    h, w = get_image_size(np.asarray(input_image), input_data_format) if not isinstance(input_image, Image.Image) \
        else (input_image.size[1], input_image.size[0])
    short, long = (w, h) if w <= h else (h, w)
    new_short, new_long = int(size), int(size * long / short)
    if max_size is not None:
        if max_size <= size:
            raise ValueError(f"max_size = {max_size} must be strictly greater than the requested size {size}")
        if new_long > max_size:
            new_short, new_long = int(max_size * new_short / new_long), max_size
    return (new_long, new_short) if w <= h else (new_short, new_long)


def resize(image: np.ndarray, size: Tuple[int, int], resample=None, reducing_gap: Optional[int] = None, data_format=None,
           return_numpy: bool = True, input_data_format=None):
    """Resize to ``size = (height, width)`` through PIL (``resample``: a PIL filter or its integer code; bilinear by
    default). Float images in [0, 1] come back as floats in [0, 1]."""
    src_fmt = ChannelDimension(input_data_format) if input_data_format is not None else infer_channel_dimension_format(np.asarray(image))
    dst_fmt = ChannelDimension(data_format) if data_format is not None else src_fmt
    arr = np.asarray(image)
    scaled = not isinstance(image, Image.Image) and _needs_rescale(arr)
    pil = to_pil_image(image, do_rescale=scaled, input_data_format=src_fmt)
    flt = _RESAMPLE.get(resample, resample) if resample is not None else Image.BILINEAR
    out = pil.resize((int(size[1]), int(size[0])), resample=flt, reducing_gap=reducing_gap)
    if not return_numpy:
        return out
    res = np.asarray(out)
    if res.ndim == 2:
        res = res[..., None]
    res = to_channel_dimension_format(res, dst_fmt, ChannelDimension.LAST)
    return res.astype(np.float32) / 255.0 if scaled else res


def normalize(image: np.ndarray, mean: Union[float, Iterable[float]], std: Union[float, Iterable[float]], data_format=None,
              input_data_format=None) -> np.ndarray:
    fmt = ChannelDimension(input_data_format) if input_data_format is not None else infer_channel_dimension_format(image)
    axis = get_channel_dimension_axis(image, fmt)
    c = image.shape[axis]
    mean = np.full(c, mean, dtype=np.float64) if np.isscalar(mean) else np.asarray(list(mean), dtype=np.float64)
    std = np.full(c, std, dtype=np.float64) if np.isscalar(std) else np.asarray(list(std), dtype=np.float64)
    if len(mean) != c or len(std) != c:
        raise ValueError(f"mean / std must have {c} elements")
    shape = [1] * image.ndim
    shape[axis] = c
    out = ((image.astype(np.float64) - mean.reshape(shape)) / std.reshape(shape)).astype(np.float32)
    return to_channel_dimension_format(out, data_format, fmt) if data_format is not None else out


def center_crop(image: np.ndarray, size: Tuple[int, int], data_format=None, input_data_format=None) -> np.ndarray:
    """Central ``(height, width)`` window; an image smaller than the window is zero-padded around its centre first."""
    fmt = ChannelDimension(input_data_format) if input_data_format is not None else infer_channel_dimension_format(image)
    out_fmt = ChannelDimension(data_format) if data_format is not None else fmt
    img = to_channel_dimension_format(image, ChannelDimension.FIRST, fmt)
    h, w = img.shape[-2:]
    ch, cw = int(size[0]), int(size[1])
    top, left = (h - ch) // 2, (w - cw) // 2
    if top < 0 or left < 0:
        nh, nw = max(h, ch), max(w, cw)
        canvas = np.zeros(img.shape[:-2] + (nh, nw), dtype=img.dtype)
        pt, pl = -(-(nh - h) // 2), -(-(nw - w) // 2)
        canvas[..., pt:pt + h, pl:pl + w] = img
        img, h, w = canvas, nh, nw
        top, left = (h - ch) // 2, (w - cw) // 2
    out = img[..., top:top + ch, left:left + cw]
    return to_channel_dimension_format(out, out_fmt, ChannelDimension.FIRST)


def pad(image: np.ndarray, padding: Union[int, Tuple[int, int], Iterable[Tuple[int, int]]], mode=PaddingMode.CONSTANT,
        constant_values: Union[float, Iterable[float]] = 0.0, data_format=None, input_data_format=None) -> np.ndarray:
    """Pad height and width: ``padding`` is one int (all sides), ``(before, after)`` for both axes, or
    ``((top, bottom), (left, right))``."""
    fmt = ChannelDimension(input_data_format) if input_data_format is not None else infer_channel_dimension_format(image)
    if isinstance(padding, (int, float)):
        hw = ((int(padding), int(padding)), (int(padding), int(padding)))
    else:
        padding = tuple(padding)
        if len(padding) == 2 and all(isinstance(p, (int, float)) for p in padding):
            hw = ((int(padding[0]), int(padding[1])), (int(padding[0]), int(padding[1])))
        elif len(padding) == 2:
            hw = (tuple(int(v) for v in padding[0]), tuple(int(v) for v in padding[1]))
        else:
            raise ValueError(f"Unsupported padding {padding}")
    lead = [(0, 0)] * (image.ndim - 3)
    widths = lead + ([(0, 0), hw[0], hw[1]] if fmt == ChannelDimension.FIRST else [hw[0], hw[1], (0, 0)])
    mode = PaddingMode(mode)
    if mode == PaddingMode.CONSTANT:
        out = np.pad(image, widths, mode="constant", constant_values=constant_values)
    else:
        out = np.pad(image, widths, mode={"reflect": "reflect", "replicate": "edge", "symmetric": "symmetric"}[mode.value])
    return to_channel_dimension_format(out, data_format, fmt) if data_format is not None else out
