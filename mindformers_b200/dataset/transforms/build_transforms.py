"""``build_transforms``: one transform or a list of them from configuration (reference
``dataset/transforms/build_transforms.py:24-70``). A list of configurations gives a list of instances, which the dataset
applies in order; ``Compose`` wraps such a list into one callable."""
from __future__ import annotations

from typing import Optional

from ...tools.register import MindFormerModuleType, MindFormerRegister
from . import vision_transforms  # noqa: F401  (registers the classes)


class Compose:
    def __init__(self, transforms):
        self.transforms = list(transforms)

    def __call__(self, x):
        for t in self.transforms:
            x = t(x)
        return x


def build_transforms(config=None, default_args: Optional[dict] = None, module_type: str = "transforms",
                     class_name: Optional[str] = None, **kwargs):
    """``config``: a mapping with ``type`` (+ constructor arguments), a list of such mappings, or None with
    ``class_name`` and keyword arguments."""
    if config is None and class_name is None:
        return None
    if config is not None:
        if isinstance(config, (list, tuple)):
            return [build_transforms(c, default_args=default_args) for c in config]
        if callable(config) and not isinstance(config, dict):
            return config
        return MindFormerRegister.get_instance_from_cfg(dict(config), MindFormerModuleType.TRANSFORMS,
                                                        default_args=default_args)
    return MindFormerRegister.get_instance(module_type, class_name, **kwargs)
