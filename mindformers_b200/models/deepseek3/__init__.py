"""DeepSeek-V3 under its reference import path (``mindformers/models/deepseek3``)."""
from ...models.families import DeepseekV3Config, DeepseekV3ForCausalLM  # noqa: F401

__all__ = ["DeepseekV3Config", "DeepseekV3ForCausalLM"]
