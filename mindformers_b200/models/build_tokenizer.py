"""``build_tokenizer`` (reference ``models/build_tokenizer.py``)."""
from ..models.tokenization import build_tokenizer  # noqa: F401

__all__ = ["build_tokenizer"]
