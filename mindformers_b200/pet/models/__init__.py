"""``LoraModel`` and friends (reference ``pet/models``)."""
from ...pet import LoraModel, PrefixTuningModel  # noqa: F401

__all__ = ["LoraModel", "PrefixTuningModel"]
