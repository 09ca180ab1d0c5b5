"""PEFT type names (reference ``pet/constants.py``)."""
from enum import Enum


class PetType(str, Enum):
    LORA = "lora"
    SLORA = "slora"
    PREFIX_TUNING = "prefixtuning"
    P_TUNING_V2 = "ptuning2"
