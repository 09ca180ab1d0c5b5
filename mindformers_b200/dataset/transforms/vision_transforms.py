"""Batched image transforms of the multimodal data pipelines.

Counterparts of the reference's ``dataset/transforms/vision_transforms.py`` (``BCHW2BHWC`` :43, ``BatchResize`` :77,
``BatchCenterCrop`` :122, ``BatchToTensor`` :167, ``BatchNormalize`` :203, ``BatchPILize`` :242 and the four
single-image transforms :282-321, which there subclass MindSpore's vision operators). Every batch transform accepts
one image or a list / stacked array of images, where an image is a ``PIL.Image``, an ``[H, W, C]`` uint8 array or a
``[C, H, W]`` float array, and returns numpy arrays (the processors convert to torch tensors at the end).
"""
from __future__ import annotations

import math
import random
from typing import List, Sequence, Union

import numpy as np
from PIL import Image

from ...tools.register import MindFormerModuleType, MindFormerRegister

_INTERP = {"nearest": Image.NEAREST, "bilinear": Image.BILINEAR, "linear": Image.BILINEAR, "bicubic": Image.BICUBIC,
           "cubic": Image.BICUBIC, "lanczos": Image.LANCZOS, "antialias": Image.LANCZOS, "area": Image.BOX}


def _as_list(images) -> tuple:
    """``(list of images, was_single)``; a 4-D array is a batch, a 3-D array or a PIL image is one image."""
    if isinstance(images, (list, tuple)):
        return list(images), False
    if isinstance(images, np.ndarray) and images.ndim == 4:
        return [images[i] for i in range(images.shape[0])], False
    return [images], True


def _to_pil(img) -> Image.Image:
    if isinstance(img, Image.Image):
        return img
    arr = np.asarray(img)
    if arr.ndim == 3 and arr.shape[0] in (1, 3, 4) and arr.shape[-1] not in (1, 3, 4):
        arr = arr.transpose(1, 2, 0)                    # CHW -> HWC
    if arr.dtype != np.uint8:
        scale = 255.0 if arr.max() <= 1.0 + 1e-6 else 1.0
        arr = np.clip(arr * scale, 0, 255).round().astype(np.uint8)
    if arr.ndim == 3 and arr.shape[-1] == 1:
        arr = arr[..., 0]
    return Image.fromarray(arr)


def _size2(size) -> tuple:
    return (int(size), int(size)) if isinstance(size, (int, float)) else (int(size[0]), int(size[1]))


@MindFormerRegister.register(MindFormerModuleType.TRANSFORMS)
class BCHW2BHWC:
    """``[B, C, H, W]`` (or a list of ``[C, H, W]``) to channel-last."""

    def __call__(self, images):
        if isinstance(images, (list, tuple)):
            return [np.asarray(i).transpose(1, 2, 0) for i in images]
        arr = np.asarray(images)
        if arr.ndim == 4:
            return arr.transpose(0, 2, 3, 1)
        if arr.ndim == 3:
            return arr.transpose(1, 2, 0)
        raise ValueError(f"expected 3 or 4 dimensions, got {arr.ndim}")


@MindFormerRegister.register(MindFormerModuleType.TRANSFORMS)
class BatchPILize:
    """Arrays to ``PIL.Image`` objects (PIL images pass through)."""

    def __call__(self, images):
        items, single = _as_list(images)
        out = [_to_pil(i) for i in items]
        return out[0] if single else out


@MindFormerRegister.register(MindFormerModuleType.TRANSFORMS)
class BatchResize:
    """Resize every image to ``image_resolution`` (an int: the SHORTER side, keeping the aspect ratio; a pair:
    ``(height, width)`` exactly)."""

    def __init__(self, image_resolution, interpolation: str = "cubic"):
        self.size = image_resolution
        self.interp = _INTERP[str(interpolation).lower()]

    def _one(self, img):
        pil = _to_pil(img)
        if isinstance(self.size, (int, float)):
            w, h = pil.size
            s = float(self.size) / min(w, h)
            new = (max(1, round(w * s)), max(1, round(h * s)))
        else:
            new = (int(self.size[1]), int(self.size[0]))
        return pil.resize(new, self.interp)

    def __call__(self, images):
        items, single = _as_list(images)
        out = [self._one(i) for i in items]
        return out[0] if single else out


@MindFormerRegister.register(MindFormerModuleType.TRANSFORMS)
class BatchCenterCrop:
    """Central ``(height, width)`` window of every image (zero padded when the image is smaller)."""

    def __init__(self, image_resolution):
        self.size = _size2(image_resolution)

    def _one(self, img):
        pil = _to_pil(img)
        w, h = pil.size
        th, tw = self.size
        left, top = int(round((w - tw) / 2.0)), int(round((h - th) / 2.0))
        return pil.crop((left, top, left + tw, top + th))

    def __call__(self, images):
        items, single = _as_list(images)
        out = [self._one(i) for i in items]
        return out[0] if single else out


@MindFormerRegister.register(MindFormerModuleType.TRANSFORMS)
class BatchToTensor:
    """PIL / uint8 HWC images to float32 ``[C, H, W]`` arrays in ``[0, 1]``."""

    def _one(self, img):
        arr = np.asarray(_to_pil(img).convert("RGB") if isinstance(img, Image.Image) else img)
        if arr.ndim == 2:
            arr = arr[..., None]
        if arr.shape[-1] in (1, 3, 4) and arr.shape[0] not in (1, 3, 4):
            arr = arr.transpose(2, 0, 1)
        elif arr.shape[-1] in (1, 3, 4) and arr.ndim == 3 and arr.shape[0] in (1, 3, 4) and arr.shape[0] != arr.shape[-1]:
            arr = arr.transpose(2, 0, 1)
        out = arr.astype(np.float32)
        return out / 255.0 if arr.dtype == np.uint8 else out

    def __call__(self, images):
        items, single = _as_list(images)
        out = [self._one(i) for i in items]
        return out[0] if single else out


@MindFormerRegister.register(MindFormerModuleType.TRANSFORMS)
class BatchNormalize:
    """``(x - mean) / std`` per channel on ``[C, H, W]`` arrays (``is_hwc=True``: channel-last input)."""

    def __init__(self, mean: Sequence[float] = (0.48145466, 0.4578275, 0.40821073),
                 std: Sequence[float] = (0.26862954, 0.26130258, 0.27577711), is_hwc: bool = False):
        self.mean = np.asarray(mean, dtype=np.float32)
        self.std = np.asarray(std, dtype=np.float32)
        self.is_hwc = is_hwc

    def _one(self, img):
        arr = np.asarray(img, dtype=np.float32)
        shape = (1, 1, -1) if self.is_hwc else (-1, 1, 1)
        return (arr - self.mean.reshape(shape)) / self.std.reshape(shape)

    def __call__(self, images):
        items, single = _as_list(images)
        out = [self._one(i) for i in items]
        return out[0] if single else out


@MindFormerRegister.register(MindFormerModuleType.TRANSFORMS)
class Resize(BatchResize):
    """Single-image resize (``size``: int = shorter side, pair = ``(height, width)``)."""

    def __init__(self, size, interpolation: str = "cubic"):
        super().__init__(size, interpolation)


@MindFormerRegister.register(MindFormerModuleType.TRANSFORMS)
class RandomResizedCrop:
    """Crop a random window covering ``scale`` of the area with an aspect ratio in ``ratio``, resize to ``size``
    (falls back to a centre crop after ten failed draws, as torchvision and MindSpore do)."""

    def __init__(self, size, scale=(0.08, 1.0), ratio=(3.0 / 4.0, 4.0 / 3.0), interpolation: str = "cubic", seed=None):
        self.size = _size2(size)
        self.scale, self.ratio = scale, ratio
        self.interp = _INTERP[str(interpolation).lower()]
        self.rng = random.Random(seed)

    def __call__(self, img):
        pil = _to_pil(img)
        w, h = pil.size
        area = w * h
        box = None
        for _ in range(10):
            target = area * self.rng.uniform(*self.scale)
            log_r = (math.log(self.ratio[0]), math.log(self.ratio[1]))
            aspect = math.exp(self.rng.uniform(*log_r))
            cw, ch = int(round(math.sqrt(target * aspect))), int(round(math.sqrt(target / aspect)))
            if 0 < cw <= w and 0 < ch <= h:
                left, top = self.rng.randint(0, w - cw), self.rng.randint(0, h - ch)
                box = (left, top, left + cw, top + ch)
                break
        if box is None:
            in_ratio = w / h
            if in_ratio < min(self.ratio):
                cw, ch = w, int(round(w / min(self.ratio)))
            elif in_ratio > max(self.ratio):
                ch, cw = h, int(round(h * max(self.ratio)))
            else:
                cw, ch = w, h
            left, top = (w - cw) // 2, (h - ch) // 2
            box = (left, top, left + cw, top + ch)
        return pil.crop(box).resize((self.size[1], self.size[0]), self.interp)


@MindFormerRegister.register(MindFormerModuleType.TRANSFORMS)
class RandomCropDecodeResize(RandomResizedCrop):
    """``RandomResizedCrop`` on an encoded image (bytes or a path): decode, crop, resize."""

    def __call__(self, img):
        if isinstance(img, (bytes, bytearray)):
            import io
            img = Image.open(io.BytesIO(img)).convert("RGB")
        elif isinstance(img, str):
            img = Image.open(img).convert("RGB")
        elif isinstance(img, np.ndarray) and img.ndim == 1:
            import io
            img = Image.open(io.BytesIO(img.tobytes())).convert("RGB")
        return super().__call__(img)


@MindFormerRegister.register(MindFormerModuleType.TRANSFORMS)
class RandomHorizontalFlip:
    """Mirror the image with probability ``prob``."""

    def __init__(self, prob: float = 0.5, seed=None):
        self.prob = prob
        self.rng = random.Random(seed)

    def __call__(self, img):
        pil = _to_pil(img)
        return pil.transpose(Image.FLIP_LEFT_RIGHT) if self.rng.random() < self.prob else pil
