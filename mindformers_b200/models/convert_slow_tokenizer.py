"""``convert_slow_tokenizer`` (reference ``models/convert_slow_tokenizer.py``)."""
from ..models.tokenizers import convert_slow_tokenizer, merges_from_ranks  # noqa: F401

__all__ = ["convert_slow_tokenizer", "merges_from_ranks"]
