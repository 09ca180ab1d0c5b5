"""String-keyed class registry used by every ``build_*`` factory.

Same surface as the reference's ``MindFormerRegister`` (``mindformers/tools/register/register.py:131``):
``register`` / ``register_cls`` / ``is_exist`` / ``get_cls`` / ``get_instance_from_cfg`` /
``get_instance`` / ``auto_register``; 27 module kinds (:102-128); classes of the Megatron-style stack
are stored under an ``mcore_`` alias when ``use_legacy`` is off (:24, :475-478).
"""
from __future__ import annotations

import importlib
import importlib.util
import inspect
import os
import sys
from typing import Any, Callable, Dict, Optional

MCORE_PREFIX = "mcore_"


class MindFormerModuleType:
    """Kinds of registrable modules."""
    CALLBACK = "callback"
    CONFIG = "config"
    CONTEXT = "context"
    DATASET = "dataset"
    DATASET_LOADER = "dataset_loader"
    DATASET_SAMPLER = "dataset_sampler"
    DATA_HANDLER = "data_handler"
    ENCODER = "encoder"
    FEATURE_EXTRACTOR = "feature_extractor"
    LOSS = "loss"
    LR = "lr"
    MASK_POLICY = "mask_policy"
    METRIC = "metric"
    MODELS = "models"
    OPTIMIZER = "optimizer"
    PIPELINE = "pipeline"
    PROCESSOR = "processor"
    TOKENIZER = "tokenizer"
    TOOLS = "tools"
    TRAINER = "trainer"
    TRANSFORMS = "transforms"
    WRAPPER = "wrapper"
    MODULES = "modules"
    BASE_LAYER = "base_layer"
    CORE = "core"
    HEAD = "head"
    GENERAL = "general"

    @classmethod
    def all(cls):
        return [v for k, v in vars(cls).items() if k.isupper() and isinstance(v, str)]


_USE_LEGACY = True


def set_use_legacy(flag: bool):
    global _USE_LEGACY
    _USE_LEGACY = bool(flag)


def is_legacy_mode() -> bool:
    return _USE_LEGACY


class MindFormerRegister:
    """Registry ``{module_type: {alias: class}}``."""
    registry: Dict[str, Dict[str, Any]] = {}

    @classmethod
    def register(cls, module_type: str = MindFormerModuleType.TOOLS, alias: Optional[str] = None,
                 legacy: bool = True, search_names=None) -> Callable:
        """Class decorator. ``legacy=False`` marks a class of the Megatron-style (mcore) stack."""
        def decorator(target):
            cls.register_cls(target, module_type, alias, legacy=legacy)
            for extra in (search_names or []):
                cls.register_cls(target, module_type, extra, legacy=legacy)
            return target
        return decorator

    @classmethod
    def register_cls(cls, register_class, module_type: str = MindFormerModuleType.TOOLS,
                     alias: Optional[str] = None, legacy: bool = True):
        name = alias or register_class.__name__
        if not legacy and module_type in (MindFormerModuleType.MODELS, MindFormerModuleType.CONFIG):
            name = MCORE_PREFIX + name
        bucket = cls.registry.setdefault(module_type, {})
        if name in bucket and bucket[name] is not register_class:
            raise KeyError(f"{name!r} is already registered as a {module_type}")
        bucket[name] = register_class
        return register_class

    @classmethod
    def _resolve(cls, module_type: str, name: str):
        bucket = cls.registry.get(module_type, {})
        if not _USE_LEGACY and module_type in (MindFormerModuleType.MODELS, MindFormerModuleType.CONFIG):
            pref = MCORE_PREFIX + name
            if pref in bucket:
                return bucket[pref]
        if name in bucket:
            return bucket[name]
        if MCORE_PREFIX + name in bucket:
            return bucket[MCORE_PREFIX + name]
        return None

    @classmethod
    def is_exist(cls, module_type: str, class_name: Optional[str] = None) -> bool:
        if class_name is None:
            return module_type in cls.registry
        return cls._resolve(module_type, class_name) is not None

    @classmethod
    def get_cls(cls, module_type: str, class_name: str):
        found = cls._resolve(module_type, class_name)
        if found is None:
            known = sorted(cls.registry.get(module_type, {}))
            raise ValueError(f"no {module_type} named {class_name!r} is registered (known: {known})")
        return found

    @classmethod
    def get_instance_from_cfg(cls, cfg: dict, module_type: str = MindFormerModuleType.TOOLS,
                              default_args: Optional[dict] = None):
        """Instantiate ``cfg['type']`` with the remaining keys (and ``default_args``) as kwargs."""
        if not isinstance(cfg, dict) or "type" not in cfg:
            raise KeyError(f"configuration {cfg!r} needs a 'type' key")
        kwargs = {k: v for k, v in cfg.items() if k != "type"}
        if default_args:
            for k, v in default_args.items():
                kwargs.setdefault(k, v)
        obj_type = cfg["type"]
        target = cls.get_cls(module_type, obj_type) if isinstance(obj_type, str) else obj_type
        try:
            return target(**kwargs)
        except TypeError as e:
            raise TypeError(f"{getattr(target, '__name__', target)}: {e}") from e

    @classmethod
    def get_instance(cls, module_type: str = MindFormerModuleType.TOOLS, class_name: Optional[str] = None,
                     **kwargs):
        if class_name is None:
            raise ValueError("class_name is required")
        return cls.get_cls(module_type, class_name)(**kwargs)

    @classmethod
    def auto_register(cls, class_reference: str, module_type: str = MindFormerModuleType.TOOLS):
        """Import ``"pkg.module.Class"`` (searched in ``$REGISTER_PATH`` too) and register it."""
        module_name, _, class_name = class_reference.rpartition(".")
        if not module_name:
            raise ValueError(f"auto_register expects 'module.Class', got {class_reference!r}")
        register_path = os.environ.get("REGISTER_PATH")
        module = None
        if register_path:
            candidate = os.path.join(register_path, *module_name.split(".")) + ".py"
            if os.path.isfile(candidate):
                spec = importlib.util.spec_from_file_location(module_name, candidate)
                module = importlib.util.module_from_spec(spec)
                sys.modules[module_name] = module
                spec.loader.exec_module(module)
            elif register_path not in sys.path:
                sys.path.insert(0, register_path)
        if module is None:
            module = importlib.import_module(module_name)
        target = getattr(module, class_name)
        if not inspect.isclass(target) and not callable(target):
            raise TypeError(f"{class_reference} is not a class")
        bucket = cls.registry.setdefault(module_type, {})
        bucket.setdefault(class_name, target)
        return target
