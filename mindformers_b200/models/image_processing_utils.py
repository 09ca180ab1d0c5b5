"""Image processor persistence and lookup (reference ``models/image_processing_utils.py:34`` ``ImageProcessingMixin``,
``:452`` ``BaseImageProcessor``; ``models/auto/image_processing_auto.py`` ``AutoImageProcessor`` /
``IMAGE_PROCESSOR_MAPPING``).

An image processor is described by ``preprocessor_config.json``: its constructor arguments plus
``image_processor_type`` (the class name). ``ImageProcessingMixin`` writes and reads that file; ``AutoImageProcessor``
picks the class the file names from the processor registry."""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Tuple

from ..models.multi_modal import BaseImageProcessor as _BaseImageProcessor
from ..tools.register import MindFormerModuleType, MindFormerRegister

IMAGE_PROCESSOR_NAME = "preprocessor_config.json"


class ImageProcessingMixin:
    """``to_dict`` / ``save_pretrained`` / ``from_pretrained`` / ``from_dict`` over ``preprocessor_config.json``."""

    def to_dict(self) -> Dict[str, Any]:
        out = {}
        for k, v in dict(getattr(self, "config", None) or {}).items():
            out[k] = list(v) if isinstance(v, tuple) else v
        out["image_processor_type"] = type(self).__name__
        return out

    def to_json_string(self) -> str:
        return json.dumps(self.to_dict(), indent=2, sort_keys=True) + "\n"

    def to_json_file(self, path: str):
        with open(path, "w", encoding="utf-8") as f:
            f.write(self.to_json_string())

    def save_pretrained(self, save_directory: str, **kwargs):
        if os.path.isfile(save_directory):
            raise ValueError(f"{save_directory} is a file, a directory is expected")
        os.makedirs(save_directory, exist_ok=True)
        path = os.path.join(save_directory, IMAGE_PROCESSOR_NAME)
        self.to_json_file(path)
        return [path]

    @classmethod
    def get_image_processor_dict(cls, name_or_dir: str, **kwargs) -> Tuple[Dict[str, Any], Dict[str, Any]]:
        path = os.path.join(name_or_dir, IMAGE_PROCESSOR_NAME) if os.path.isdir(name_or_dir) else name_or_dir
        if not os.path.isfile(path):
            raise EnvironmentError(f"no {IMAGE_PROCESSOR_NAME} at {name_or_dir}")
        with open(path, encoding="utf-8") as f:
            return json.load(f), kwargs

    @classmethod
    def from_dict(cls, image_processor_dict: Dict[str, Any], **kwargs):
        d = {k: v for k, v in image_processor_dict.items() if k != "image_processor_type"}
        return_unused = kwargs.pop("return_unused_kwargs", False)
        d.update({k: kwargs.pop(k) for k in list(kwargs) if k in d})
        obj = cls(**d)
        return (obj, kwargs) if return_unused else obj

    @classmethod
    def from_pretrained(cls, name_or_dir: str, **kwargs):
        d, kwargs = cls.get_image_processor_dict(name_or_dir, **kwargs)
        return cls.from_dict(d, **kwargs)

    @classmethod
    def from_json_file(cls, path: str):
        with open(path, encoding="utf-8") as f:
            return cls.from_dict(json.load(f))

    def __repr__(self):
        return f"{type(self).__name__} {self.to_json_string()}"


class BaseImageProcessor(ImageProcessingMixin, _BaseImageProcessor):
    """``BaseImageProcessor`` with persistence (the class user processors derive from)."""


class _ImageProcessorMapping(dict):
    """``class name -> image processor class`` over the processor registry, evaluated at lookup time."""

    @staticmethod
    def _table():
        out = {}
        for name, cls in MindFormerRegister.registry.get(MindFormerModuleType.PROCESSOR, {}).items():
            if isinstance(cls, type) and issubclass(cls, _BaseImageProcessor):
                out[name] = cls
        return out

    def __getitem__(self, key):
        return self._table()[key]

    def __contains__(self, key):
        return key in self._table()

    def __iter__(self):
        return iter(self._table())

    def __len__(self):
        return len(self._table())

    def keys(self):
        return self._table().keys()

    def items(self):
        return self._table().items()

    def values(self):
        return self._table().values()

    def get(self, key, default=None):
        return self._table().get(key, default)

    def register(self, key, value, exist_ok: bool = False):
        if key in self._table() and not exist_ok:
            raise ValueError(f"{key!r} is already registered")
        MindFormerRegister.register_cls(value, MindFormerModuleType.PROCESSOR, alias=key)


IMAGE_PROCESSOR_MAPPING = _ImageProcessorMapping()


class AutoImageProcessor:
    """``from_pretrained(directory)`` builds the image processor class that ``preprocessor_config.json`` names."""

    def __init__(self):
        raise EnvironmentError("AutoImageProcessor is built with AutoImageProcessor.from_pretrained(directory)")

    @classmethod
    def from_pretrained(cls, name_or_dir: str, **kwargs):
        d, kwargs = ImageProcessingMixin.get_image_processor_dict(name_or_dir, **kwargs)
        name = d.get("image_processor_type") or d.get("type")
        if name not in IMAGE_PROCESSOR_MAPPING:
            raise ValueError(f"unknown image processor type {name!r}; known: {sorted(IMAGE_PROCESSOR_MAPPING)}")
        target = IMAGE_PROCESSOR_MAPPING[name]
        args = {k: v for k, v in d.items() if k not in ("image_processor_type", "type")}
        args.update(kwargs)
        return target(**args)

    @staticmethod
    def register(name_or_config, image_processor_class, exist_ok: bool = False):
        key = name_or_config if isinstance(name_or_config, str) else image_processor_class.__name__
        IMAGE_PROCESSOR_MAPPING.register(key, image_processor_class, exist_ok=exist_ok)


__all__ = ["AutoImageProcessor", "BaseImageProcessor", "IMAGE_PROCESSOR_MAPPING", "IMAGE_PROCESSOR_NAME", "ImageProcessingMixin"]
