from .pet_config import LoraConfig, PetConfig, PrefixTuningConfig, Ptuning2Config, SLoraConfig
from .lora import (ColumnParallelLinearWithLoRA, LoraAdapter, LoraModel, LoRALinear, RowParallelLinearWithLoRA,
                   lora_state_dict, merge_lora_weights)
from .slora import SLoraAdapter, SLoraLinear
from .prompt import PrefixEncoder, PrefixTuningModel
from .pet_model import get_pet_model, is_supported_pet_type
