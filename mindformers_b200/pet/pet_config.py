"""Parameter-efficient tuning configurations (``mindformers/pet/pet_config.py``)."""
from __future__ import annotations

from dataclasses import asdict, dataclass, field
from typing import List, Optional

from ..tools.register.register import MindFormerModuleType, MindFormerRegister


@dataclass
class PetConfig:
    """Base of the parameter-efficient tuning configurations (reference ``pet/pet_config.py``): ``pet_type`` selects
    the adapter."""

    pet_type: Optional[str] = None

    def to_dict(self):
        return asdict(self)


@MindFormerRegister.register(MindFormerModuleType.CONFIG, alias="LoraConfig")
@dataclass
class LoraConfig(PetConfig):
    """``target_modules`` is a regular expression matched against module names (the reference's default for Llama is
    ``'.*wq|.*wk|.*wv|.*wo'``; with fused projections use ``'.*linear_qkv|.*linear_proj'``)."""
    pet_type: str = "lora"
    lora_rank: int = 8
    lora_alpha: int = 16
    lora_dropout: float = 0.0
    lora_a_init: str = "normal"
    lora_b_init: str = "zero"
    param_init_type: str = "float32"
    compute_dtype: str = "bfloat16"
    target_modules: str = ".*linear_qkv|.*linear_proj"
    exclude_layers: Optional[List[str]] = None
    freeze_include: Optional[List[str]] = None
    freeze_exclude: Optional[List[str]] = None


@MindFormerRegister.register(MindFormerModuleType.CONFIG, alias="SLoraConfig")
@dataclass
class SLoraConfig(PetConfig):
    """Multi-adapter LoRA serving: directory of adapters, maximum rank, target modules."""

    pet_type: str = "slora"
    lora_num: int = 1
    lora_rank: int = 8
    lora_alpha: int = 16
    lora_dropout: float = 0.0
    target_modules: str = ".*linear_qkv|.*linear_proj"
    adapter_path: Optional[str] = None


@MindFormerRegister.register(MindFormerModuleType.CONFIG, alias="PrefixTuningConfig")
@dataclass
class PrefixTuningConfig(PetConfig):
    """Prefix tuning: ``prefix_token_num`` trainable key / value vectors per layer."""

    pet_type: str = "prefixtuning"
    prefix_token_num: int = 16
    mid_dim: int = 512
    dropout_rate: float = 0.0


@MindFormerRegister.register(MindFormerModuleType.CONFIG, alias="Ptuning2Config")
@dataclass
class Ptuning2Config(PetConfig):
    """P-Tuning v2: ``pre_seq_len`` trainable prefix tokens through an optional re-parameterisation MLP."""

    pet_type: str = "ptuning2"
    pre_seq_len: int = 16
    prefix_projection: bool = False
    projection_dim: int = 128
    dropout_prob: float = 0.0
