"""Processors: objects that turn raw inputs (text, images) into model input tensors and can be saved beside a model.

Reference: ``mindformers/models/processing_utils.py`` (``ProcessorMixin:72``: attributes named in ``attributes``,
``save_pretrained`` / ``from_pretrained`` over ``preprocessor_config.json`` and the tokenizer files),
``models/base_processor.py`` (``BaseProcessor``: ``__call__(image_input=…, text_input=…)`` with ``max_length``,
``padding``, ``return_tensors``), ``models/build_processor.py``, ``models/llama/llama_processor.py``,
``models/glm2/glm_processor.py``.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Optional

from ..tools.register import MindFormerModuleType, MindFormerRegister

PROCESSOR_CONFIG = "preprocessor_config.json"


class ProcessorMixin:
    """Holds the sub-processors listed in ``attributes`` (``tokenizer``, ``image_processor`` …) and persists them."""
    attributes: List[str] = ["tokenizer"]

    def __init__(self, *args, **kwargs):
        for name, value in zip(self.attributes, args):
            kwargs.setdefault(name, value)
        for name in self.attributes:
            setattr(self, name, kwargs.pop(name, None))
        self.config: Dict[str, Any] = kwargs

    def to_dict(self) -> Dict[str, Any]:
        out = {"processor_class": type(self).__name__}
        out.update({k: v for k, v in self.config.items() if isinstance(v, (str, int, float, bool, list, dict, type(None)))})
        for name in self.attributes:
            sub = getattr(self, name, None)
            if sub is not None and name != "tokenizer" and hasattr(sub, "config"):
                out[name] = {"type": type(sub).__name__, **{k: (list(v) if isinstance(v, tuple) else v)
                                                            for k, v in sub.config.items()}}
        return out

    def save_pretrained(self, save_directory: str):
        os.makedirs(save_directory, exist_ok=True)
        tok = getattr(self, "tokenizer", None)
        if tok is not None and hasattr(tok, "save_pretrained"):
            tok.save_pretrained(save_directory)
        with open(os.path.join(save_directory, PROCESSOR_CONFIG), "w", encoding="utf-8") as f:
            json.dump(self.to_dict(), f, indent=2, default=str)

    @classmethod
    def from_pretrained(cls, directory: str, **kwargs):
        cfg: Dict[str, Any] = {}
        path = os.path.join(directory, PROCESSOR_CONFIG)
        if os.path.exists(path):
            with open(path, "r", encoding="utf-8") as f:
                cfg = json.load(f)
        cfg.pop("processor_class", None)
        subs = {}
        for name in cls.attributes:
            if name == "tokenizer":
                from .auto import AutoTokenizer
                subs[name] = kwargs.pop("tokenizer", None) or AutoTokenizer.from_pretrained(directory)
            elif isinstance(cfg.get(name), dict):
                sub_cfg = dict(cfg.pop(name))
                subs[name] = MindFormerRegister.get_instance_from_cfg(sub_cfg, MindFormerModuleType.PROCESSOR)
        cfg.update(kwargs)
        return cls(**subs, **cfg)


class BaseProcessor(ProcessorMixin):
    """``processor(text_input=…, image_input=…)`` → dict with ``text`` (token ids), ``attention_mask`` and, when an
    image processor is attached, ``image``."""
    attributes = ["tokenizer", "image_processor"]

    def __init__(self, tokenizer=None, image_processor=None, max_length: int = 128, padding: str = "max_length",
                 return_tensors: Optional[str] = "pt", **kwargs):
        super().__init__(tokenizer=tokenizer, image_processor=image_processor, max_length=max_length, padding=padding,
                         return_tensors=return_tensors, **kwargs)
        self.max_length, self.padding, self.return_tensors = max_length, padding, return_tensors

    def __call__(self, image_input=None, text_input=None, **kwargs) -> Dict[str, Any]:
        out: Dict[str, Any] = {}
        if image_input is not None:
            if self.image_processor is None:
                raise ValueError(f"{type(self).__name__} has no image_processor")
            out["image"] = self.image_processor(image_input)
        if text_input is not None:
            if self.tokenizer is None:
                raise ValueError(f"{type(self).__name__} has no tokenizer")
            enc = self.tokenizer(text_input, padding=self.padding, max_length=self.max_length, truncation=True,
                                 return_tensors=self.return_tensors)
            out["text"] = enc["input_ids"]
            if "attention_mask" in enc:
                out["attention_mask"] = enc["attention_mask"]
        return out


@MindFormerRegister.register(MindFormerModuleType.PROCESSOR)
class LlamaProcessor(BaseProcessor):
    """Tokenizer wrapper returning padded ``input_ids`` tensors (reference ``models/llama/llama_processor.py``)."""

    attributes = ["tokenizer"]

    def __init__(self, tokenizer=None, max_length: int = 128, padding: str = "max_length", return_tensors="pt", **kw):
        super().__init__(tokenizer=tokenizer, max_length=max_length, padding=padding, return_tensors=return_tensors, **kw)


@MindFormerRegister.register(MindFormerModuleType.PROCESSOR)
class GLMProcessor(LlamaProcessor):
    """GLM tokenizers pad on the left and add ``position_ids``; the processor passes them through."""

    def __call__(self, image_input=None, text_input=None, **kwargs):
        out = super().__call__(image_input, text_input, **kwargs)
        if text_input is not None and self.tokenizer is not None and "position_ids" in getattr(
                self.tokenizer, "model_input_names", []):
            enc = self.tokenizer(text_input, padding=self.padding, max_length=self.max_length, truncation=True,
                                 return_tensors=self.return_tensors)
            if "position_ids" in enc:
                out["position_ids"] = enc["position_ids"]
        return out


def build_processor(config: Optional[dict] = None, default_args: Optional[dict] = None, **kwargs):
    """``{"type": "LlamaProcessor", "tokenizer": {...}, "image_processor": {...}, "max_length": …}`` → processor."""
    if config is None:
        return None
    cfg = dict(config)
    cfg.update(kwargs)
    if default_args:
        for k, v in default_args.items():
            cfg.setdefault(k, v)
    if isinstance(cfg.get("tokenizer"), dict):
        from .tokenization import build_tokenizer
        cfg["tokenizer"] = build_tokenizer(cfg["tokenizer"])
    if isinstance(cfg.get("image_processor"), dict):
        cfg["image_processor"] = MindFormerRegister.get_instance_from_cfg(dict(cfg["image_processor"]),
                                                                          MindFormerModuleType.PROCESSOR)
    return MindFormerRegister.get_instance_from_cfg(cfg, MindFormerModuleType.PROCESSOR)
