"""``PretrainedConfig``: HF-compatible model configuration (dict round trip, ``from_pretrained`` / ``save_pretrained``).

Reference: ``models/configuration_utils.py`` / ``models/base_config.py``. A configuration keeps HF key names
(``num_hidden_layers`` …); ``convert_to_transformer_config`` maps them to the Megatron-named fields the layers read.
"""
from __future__ import annotations

import copy
import json
import os
from typing import Optional

import yaml

CONFIG_NAME = "config.json"


class PretrainedConfig:
    """Hugging Face compatible model configuration (reference ``models/configuration_utils.py``): attribute access to
    the keys of ``config.json``, class defaults via ``default_values()``, ``from_pretrained`` / ``from_dict`` /
    ``from_json_file`` / ``to_dict`` / ``save_pretrained``; unknown keys are kept."""

    model_type: str = ""
    is_mla: bool = False

    def __init__(self, **kwargs):
        self.parallel_config = kwargs.pop("parallel_config", None)
        for k, v in self.default_values().items():
            setattr(self, k, copy.deepcopy(v))
        for k, v in kwargs.items():
            setattr(self, k, v)
        if not getattr(self, "model_type", None):
            self.model_type = type(self).model_type

    @classmethod
    def default_values(cls) -> dict:
        return {}

    def to_dict(self) -> dict:
        out = {}
        for k, v in vars(self).items():
            if k.startswith("_") or callable(v):
                continue
            if hasattr(v, "to_dict"):
                v = v.to_dict()
            out[k] = copy.deepcopy(v)
        out["model_type"] = self.model_type
        return out

    def to_json_string(self) -> str:
        return json.dumps(self.to_dict(), indent=2, sort_keys=True, default=str)

    def save_pretrained(self, save_directory: str, save_name: str = "mindspore_model"):
        os.makedirs(save_directory, exist_ok=True)
        with open(os.path.join(save_directory, CONFIG_NAME), "w") as f:
            f.write(self.to_json_string())
        with open(os.path.join(save_directory, save_name + ".yaml"), "w") as f:
            yaml.safe_dump({"model": {"model_config": json.loads(self.to_json_string()),
                                      "arch": {"type": getattr(self, "architectures", [None])[0]}}}, f)

    @classmethod
    def from_dict(cls, config_dict: dict, **kwargs) -> "PretrainedConfig":
        d = dict(config_dict)
        d.update(kwargs)
        d.pop("type", None)
        return cls(**d)

    @classmethod
    def from_json_file(cls, path: str) -> "PretrainedConfig":
        with open(path) as f:
            return cls.from_dict(json.load(f))

    @classmethod
    def from_pretrained(cls, name_or_path: str, **kwargs) -> "PretrainedConfig":
        """Directory with ``config.json``, a ``.json`` file, or a YAML with ``model.model_config``."""
        path = name_or_path
        if os.path.isdir(path):
            path = os.path.join(path, CONFIG_NAME)
        if not os.path.exists(path):
            raise FileNotFoundError(f"no configuration found at {name_or_path}")
        if path.endswith((".yaml", ".yml")):
            with open(path) as f:
                data = yaml.safe_load(f)
            d = dict((data.get("model") or {}).get("model_config") or data)
        else:
            with open(path) as f:
                d = json.load(f)
        return cls.from_dict(d, **kwargs)

    def __repr__(self):
        return f"{type(self).__name__} {self.to_json_string()}"

    def update(self, d: dict):
        for k, v in d.items():
            setattr(self, k, v)
