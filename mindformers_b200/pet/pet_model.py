"""``get_pet_model(model, pet_config)``: dispatch on ``pet_type`` (``mindformers/pet/pet_model.py``)."""
from __future__ import annotations

from .lora import LoraModel
from .pet_config import LoraConfig, PrefixTuningConfig, Ptuning2Config, SLoraConfig
from .prompt import PrefixTuningModel
from .slora import SLoraAdapter

_TYPES = {"lora": LoraConfig, "slora": SLoraConfig, "prefixtuning": PrefixTuningConfig, "ptuning2": Ptuning2Config}


def is_supported_pet_type(pet_type: str) -> bool:
    return str(pet_type).lower() in _TYPES


def get_pet_model(model, pet_config):
    if isinstance(pet_config, dict):
        d = dict(pet_config)
        kind = str(d.pop("pet_type", d.pop("type", "lora"))).lower()
        if kind not in _TYPES:
            raise ValueError(f"pet_type {kind!r} is not supported; choose from {sorted(_TYPES)}")
        pet_config = _TYPES[kind](**d)
    kind = pet_config.pet_type.lower()
    if kind == "lora":
        return LoraModel(pet_config, model)
    if kind == "slora":
        model.slora = SLoraAdapter(model, pet_config)
        return model
    if kind in ("prefixtuning", "ptuning2"):
        return PrefixTuningModel(pet_config, model)
    raise ValueError(f"pet_type {kind!r} is not supported")
