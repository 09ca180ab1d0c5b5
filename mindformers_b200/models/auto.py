"""``AutoConfig`` / ``AutoModel`` / ``AutoModelForCausalLM`` / ``AutoTokenizer`` / ``AutoProcessor``.

Reference: ``models/auto/*`` (``auto_factory.py:217-764``, ``configuration_auto.py:189``, ``tokenization_auto.py``).
Resolution order: explicit ``model_type`` / ``architectures`` of a ``config.json`` or YAML ``model.model_config``,
then user registrations (``register``).
"""
from __future__ import annotations

import json
import os
from typing import Optional

import yaml

from ..tools.register import MindFormerConfig, MindFormerModuleType, MindFormerRegister
from .configuration_utils import PretrainedConfig
from .families import MODEL_TYPE_TO_CLASSES
from .presets import PRESETS, get_preset

_EXTRA = {}


def _read_config_dict(path: str) -> dict:
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    if path.endswith((".yaml", ".yml")):
        cfg = MindFormerConfig(path)
        d = dict((cfg.get("model") or {}).get("model_config") or {})
        arch = ((cfg.get("model") or {}).get("arch") or {}).get("type")
        if arch and "architectures" not in d:
            d["architectures"] = [arch]
        return d
    with open(path) as f:
        return json.load(f)


def _classes_for(d: dict):
    mt = d.get("model_type") or d.get("type")
    if mt in _EXTRA:
        return _EXTRA[mt]
    if mt in MODEL_TYPE_TO_CLASSES:
        return MODEL_TYPE_TO_CLASSES[mt]
    for arch in d.get("architectures") or []:
        if MindFormerRegister.is_exist(MindFormerModuleType.MODELS, arch):
            m = MindFormerRegister.get_cls(MindFormerModuleType.MODELS, arch)
            return m.config_class, m
    if isinstance(mt, str):
        for key, val in MODEL_TYPE_TO_CLASSES.items():
            if key in mt.lower():
                return val
    raise ValueError(f"cannot determine the model family of configuration with model_type={mt!r}")


class AutoConfig:
    @staticmethod
    def from_pretrained(name_or_path: str, **kwargs) -> PretrainedConfig:
        if name_or_path in PRESETS:
            d = get_preset(name_or_path)
        else:
            d = _read_config_dict(name_or_path)
        cfg_cls, _ = _classes_for(d)
        return cfg_cls.from_dict(d, **kwargs)

    @staticmethod
    def for_model(model_type: str, **kwargs) -> PretrainedConfig:
        return _classes_for({"model_type": model_type})[0](**kwargs)

    @staticmethod
    def register(model_type: str, config_cls, model_cls=None):
        _EXTRA[model_type] = (config_cls, model_cls)


class AutoModel:
    @staticmethod
    def from_config(config, **kwargs):
        """``config``: a ``PretrainedConfig``, a dict, a preset name, or a YAML / JSON path."""
        if isinstance(config, str):
            config = AutoConfig.from_pretrained(config)
        elif isinstance(config, dict):
            config = _classes_for(config)[0].from_dict(config)
        _, model_cls = _classes_for(config.to_dict())
        return model_cls(config, **kwargs)

    @staticmethod
    def from_pretrained(name_or_dir: str, **kwargs):
        config = kwargs.pop("config", None) or AutoConfig.from_pretrained(name_or_dir)
        _, model_cls = _classes_for(config.to_dict())
        if name_or_dir in PRESETS:
            return model_cls(config, **kwargs)
        return model_cls.from_pretrained(name_or_dir, config=config, **kwargs)

    @staticmethod
    def register(config_cls, model_cls, model_type: Optional[str] = None):
        _EXTRA[model_type or config_cls.model_type] = (config_cls, model_cls)


AutoModelForCausalLM = AutoModel


class AutoTokenizer:
    """Loads a tokenizer directory (``tokenizer.json`` / sentencepiece / tiktoken files) through ``transformers``;
    ``ByteTokenizer`` is the dependency-free fallback used by tests and ``run_check``."""

    @staticmethod
    def from_pretrained(name_or_dir: str, **kwargs):
        if name_or_dir in ("byte", "ByteTokenizer"):
            from .tokenization import ByteTokenizer
            return ByteTokenizer()
        if not os.path.exists(name_or_dir):
            raise FileNotFoundError(f"tokenizer directory {name_or_dir} does not exist (no hub access offline)")
        from transformers import AutoTokenizer as _HF
        return _HF.from_pretrained(name_or_dir, local_files_only=True, **kwargs)

    @staticmethod
    def register(*args, **kwargs):
        from transformers import AutoTokenizer as _HF
        return _HF.register(*args, **kwargs)


class AutoProcessor:
    @staticmethod
    def from_pretrained(name_or_dir: str, **kwargs):
        from .tokenization import TextProcessor
        return TextProcessor(AutoTokenizer.from_pretrained(name_or_dir, **kwargs), **kwargs)
