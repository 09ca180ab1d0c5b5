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


def _auto_map_classes(path: str):
    """``(config class, model class)`` named by the ``auto_map`` of a model directory's ``config.json`` (classes that
    live in Python files of that directory), or None. Either entry may be None when the map does not name it."""
    if not isinstance(path, str) or not os.path.isdir(path) or not os.path.exists(os.path.join(path, "config.json")):
        return None
    amap = _read_config_dict(path).get("auto_map") or {}
    if not amap:
        return None
    from ..tools.hub import get_class_from_dynamic_module
    cfg_ref = amap.get("AutoConfig")
    model_ref = amap.get("AutoModelForCausalLM") or amap.get("AutoModel")
    cfg_cls = get_class_from_dynamic_module(cfg_ref, path) if cfg_ref else None
    model_cls = get_class_from_dynamic_module(model_ref, path) if model_ref else None
    if cfg_cls is None and model_cls is not None:
        cfg_cls = getattr(model_cls, "config_class", None)
    return cfg_cls, model_cls


class AutoConfig:
    """Resolves a configuration class from a directory (``config.json`` ``model_type`` / ``auto_map``), a preset name or a
    YAML file (reference ``models/auto/configuration_auto.py:189``): ``from_pretrained(name_or_path)``, ``for_model(model_type)``."""

    @staticmethod
    def from_pretrained(name_or_path: str, **kwargs) -> PretrainedConfig:
        dyn = _auto_map_classes(name_or_path)
        if dyn is not None and dyn[0] is not None:
            return dyn[0].from_dict(_read_config_dict(name_or_path), **kwargs)
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
    """Builds the model class registered for a configuration (reference ``models/auto/auto_factory.py:217,764``):
    ``from_config(config)`` with random weights, ``from_pretrained(directory)`` with the weights of a Hugging Face style
    or framework directory. ``AutoModelForCausalLM`` is the same class: every registered model is a causal LM."""

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
        dyn = _auto_map_classes(name_or_dir)
        if dyn is not None and dyn[1] is not None:
            cfg_cls, model_cls = dyn
            config = kwargs.pop("config", None) or cfg_cls.from_dict(_read_config_dict(name_or_dir))
            return model_cls.from_pretrained(name_or_dir, config=config, **kwargs) if hasattr(
                model_cls, "from_pretrained") else model_cls(config, **kwargs)
        config = kwargs.pop("config", None) or AutoConfig.from_pretrained(name_or_dir)
        _, model_cls = _classes_for(config.to_dict())
        if name_or_dir in PRESETS:
            return model_cls(config, **kwargs)
        return model_cls.from_pretrained(name_or_dir, config=config, **kwargs)

    @staticmethod
    def register(config_cls, model_cls, model_type: Optional[str] = None):
        _EXTRA[model_type or config_cls.model_type] = (config_cls, model_cls)


AutoModelForCausalLM = AutoModel
# The reference keeps one factory per head type (``models/auto/modeling_auto.py``: ``AutoModelForPreTraining``,
# ``AutoModelWithLMHead``, ``AutoModelForMaskGeneration`` ...). Every registered architecture is a causal language model,
# so the head-specific factories resolve to the same classes.
AutoModelForPreTraining = AutoModel
AutoModelWithLMHead = AutoModel
AutoModelForMaskGeneration = AutoModel


class AutoTokenizer:
    """Picks the tokenizer class of a directory (reference ``models/auto/tokenization_auto.py``).

    Order: ``tokenizer_class`` of ``tokenizer_config.json`` → ``model_type`` of ``config.json`` → the vocabulary
    files present (``tokenizer.json`` → fast, ``vocab.json`` → Qwen2 BPE, ``tokenizer.model`` → sentencepiece, or a
    tiktoken rank file when it is not a sentencepiece proto). ``use_hf=True`` hands the directory to
    ``transformers`` instead. ``"byte"`` gives the file-less ``ByteTokenizer``.
    """
    _extra: dict = {}

    @classmethod
    def _resolve(cls, directory: str):
        from . import tokenizers as T
        table = dict(T.TOKENIZER_CLASSES)
        table.update(cls._extra)
        name = None
        cfg_path = os.path.join(directory, "tokenizer_config.json")
        if os.path.exists(cfg_path):
            with open(cfg_path, "r", encoding="utf-8") as f:
                name = json.load(f).get("tokenizer_class")
        has = lambda f: os.path.exists(os.path.join(directory, f))
        if name in table and all(has(table[name].vocab_files_names[k]) for k in table[name].required_vocab_files()):
            return table[name]
        if has("tokenizer.json"):
            return T.LlamaTokenizerFast
        model_type = None
        if has("config.json"):
            with open(os.path.join(directory, "config.json"), "r", encoding="utf-8") as f:
                model_type = json.load(f).get("model_type")
        if model_type in T.TOKENIZER_BY_MODEL_TYPE:
            cand = table[T.TOKENIZER_BY_MODEL_TYPE[model_type]]
            if all(has(cand.vocab_files_names[k]) for k in cand.required_vocab_files()):
                return cand
        if has("vocab.json"):
            return T.Qwen2Tokenizer
        if has("tokenizer.model"):
            with open(os.path.join(directory, "tokenizer.model"), "rb") as f:
                head = f.read(64)
            tiktoken_like = b" " in head and all(32 <= b < 127 or b in (10, 13) for b in head)
            return T.Llama3Tokenizer if tiktoken_like else T.LlamaTokenizer
        raise FileNotFoundError(f"{directory}: no tokenizer.json, vocab.json or tokenizer.model")

    @classmethod
    def from_pretrained(cls, name_or_dir: str, use_hf: bool = False, **kwargs):
        if name_or_dir in ("byte", "ByteTokenizer"):
            from .tokenization import ByteTokenizer
            return ByteTokenizer()
        if not os.path.exists(name_or_dir):
            raise FileNotFoundError(f"tokenizer directory {name_or_dir} does not exist (no hub access offline)")
        if use_hf:
            from transformers import AutoTokenizer as _HF
            return _HF.from_pretrained(name_or_dir, local_files_only=True, **kwargs)
        if os.path.isfile(name_or_dir):
            directory = os.path.dirname(name_or_dir) or "."
            return cls._resolve(directory).from_pretrained(name_or_dir, **kwargs)
        cfg_path = os.path.join(name_or_dir, "tokenizer_config.json")
        if os.path.exists(cfg_path):
            with open(cfg_path, "r", encoding="utf-8") as f:
                if json.load(f).get("tokenizer_class") == "ByteTokenizer":
                    from .tokenization import ByteTokenizer
                    return ByteTokenizer()
        return cls._resolve(name_or_dir).from_pretrained(name_or_dir, **kwargs)

    @classmethod
    def register(cls, name_or_config, tokenizer_class=None, **kwargs):
        """``register("MyTokenizer", MyTokenizer)`` or ``register(ConfigClass, MyTokenizer)``."""
        if tokenizer_class is None:
            tokenizer_class, name_or_config = name_or_config, name_or_config.__name__
        key = name_or_config if isinstance(name_or_config, str) else tokenizer_class.__name__
        cls._extra[key] = tokenizer_class
        return tokenizer_class


class AutoProcessor:
    """Processor of a directory: the class named in ``preprocessor_config.json`` (registry lookup), else a text
    processor around the directory's tokenizer."""

    @staticmethod
    def from_pretrained(name_or_dir: str, **kwargs):
        path = os.path.join(name_or_dir, "preprocessor_config.json")
        if os.path.exists(path):
            with open(path, "r", encoding="utf-8") as f:
                name = json.load(f).get("processor_class")
            if name and MindFormerRegister.is_exist(MindFormerModuleType.PROCESSOR, name):
                return MindFormerRegister.get_cls(MindFormerModuleType.PROCESSOR, name).from_pretrained(name_or_dir, **kwargs)
        from .processing_utils import LlamaProcessor
        return LlamaProcessor(AutoTokenizer.from_pretrained(name_or_dir), **kwargs)


AutoImageProcessor = AutoProcessor


class _LazyMapping(dict):
    """Read-only view ``key -> class`` over the family table and the user registrations, evaluated at lookup time
    (reference ``models/auto/configuration_auto.py`` ``_LazyConfigMapping``, ``auto_factory.py`` ``_LazyAutoMapping``)."""

    def __init__(self, pick):
        super().__init__()
        self._pick = pick

    def _table(self):
        out = {}
        for key, pair in {**MODEL_TYPE_TO_CLASSES, **_EXTRA}.items():
            val = self._pick(key, pair)
            if val is not None:
                out[key] = val
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

    def values(self):
        return self._table().values()

    def items(self):
        return self._table().items()

    def get(self, key, default=None):
        return self._table().get(key, default)

    def register(self, key, value, exist_ok: bool = False):
        if key in self._table() and not exist_ok:
            raise ValueError(f"{key!r} is already registered")
        cfg, model = _EXTRA.get(key, MODEL_TYPE_TO_CLASSES.get(key, (None, None)))
        _EXTRA[key] = (value, model) if self._pick(key, (value, None)) is value else (cfg, model)


def _tokenizer_for(key, pair):
    from . import tokenizers as T
    name = T.TOKENIZER_BY_MODEL_TYPE.get(key)
    return T.TOKENIZER_CLASSES.get(name) if name else None


CONFIG_MAPPING = _LazyMapping(lambda key, pair: pair[0])
CONFIG_MAPPING_NAMES = {k: v[0].__name__ for k, v in MODEL_TYPE_TO_CLASSES.items()}
TOKENIZER_MAPPING = _LazyMapping(_tokenizer_for)
from .image_processing_utils import IMAGE_PROCESSOR_MAPPING, AutoImageProcessor  # noqa: E402,F401


def is_experimental_mode(path) -> bool:
    """Whether ``path`` is a model directory / repository name (the ``from_pretrained`` route of the reference that reads
    ``config.json``) rather than a YAML file or a name of the built-in support list."""
    if not isinstance(path, str):
        return False
    if os.path.isdir(path):
        return not any(f.endswith((".yaml", ".yml")) for f in os.listdir(path))
    return not path.endswith((".yaml", ".yml")) and path not in PRESETS and "/" in path


def config_class_to_model_type(config_class_name: str):
    """``"LlamaConfig"`` → ``"llama"``; None for an unknown class name."""
    for key, pair in {**MODEL_TYPE_TO_CLASSES, **_EXTRA}.items():
        if pair[0] is not None and pair[0].__name__ == config_class_name:
            return key
    return None


def tokenizer_class_from_name(class_name: str):
    from . import tokenizers as T
    return T.TOKENIZER_CLASSES.get(class_name) or (
        MindFormerRegister.get_cls(MindFormerModuleType.TOKENIZER, class_name)
        if MindFormerRegister.is_exist(MindFormerModuleType.TOKENIZER, class_name) else None)


def image_processor_class_from_name(class_name: str):
    return IMAGE_PROCESSOR_MAPPING.get(class_name)


def processor_class_from_name(class_name: str):
    return (MindFormerRegister.get_cls(MindFormerModuleType.PROCESSOR, class_name)
            if MindFormerRegister.is_exist(MindFormerModuleType.PROCESSOR, class_name) else None)


def _json_of(directory: str, name: str) -> dict:
    path = os.path.join(directory, name)
    if not os.path.isfile(path):
        return {}
    with open(path, encoding="utf-8") as f:
        return json.load(f)


def get_tokenizer_config(name_or_dir: str, **kwargs) -> dict:
    """Contents of ``tokenizer_config.json`` of a model directory ({} when there is none)."""
    return _json_of(name_or_dir, "tokenizer_config.json")


def get_image_processor_config(name_or_dir: str, **kwargs) -> dict:
    """Contents of ``preprocessor_config.json`` of a model directory ({} when there is none)."""
    return _json_of(name_or_dir, "preprocessor_config.json")


from .._submodules import alias_children as _alias_children  # noqa: E402

_alias_children(__name__, ("auto_factory", "configuration_auto", "image_processing_auto", "modeling_auto", "processing_auto",
                           "tokenization_auto"))
