"""Tokenizer base types (reference ``models/tokenization_utils_base.py``)."""
from ..models.tokenization_utils import AddedToken, BatchEncoding, PreTrainedTokenizer  # noqa: F401
PreTrainedTokenizerBase = PreTrainedTokenizer

__all__ = ["AddedToken", "BatchEncoding", "PreTrainedTokenizer"]
