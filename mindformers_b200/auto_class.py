"""Older import path of the Auto classes (reference ``mindformers/auto_class.py``: ``AutoConfig``, ``AutoModel``, ``AutoProcessor``, ``AutoTokenizer`` resolved from YAML names or directories)."""
from .models.auto import AutoConfig, AutoModel, AutoModelForCausalLM, AutoProcessor, AutoTokenizer  # noqa: F401

__all__ = ["AutoConfig", "AutoModel", "AutoModelForCausalLM", "AutoProcessor", "AutoTokenizer"]
