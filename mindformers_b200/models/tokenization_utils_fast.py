"""``PreTrainedTokenizerFast`` (reference ``models/tokenization_utils_fast.py``)."""
from ..models.tokenizers import PreTrainedTokenizerFast  # noqa: F401

__all__ = ["PreTrainedTokenizerFast"]
