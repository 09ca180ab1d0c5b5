"""PEFT helpers (reference ``pet/utils.py``)."""
from ..pet import is_supported_pet_type, lora_state_dict, merge_lora_weights  # noqa: F401

__all__ = ["is_supported_pet_type", "lora_state_dict", "merge_lora_weights"]
