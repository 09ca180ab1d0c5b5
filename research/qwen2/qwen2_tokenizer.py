"""``Qwen2Tokenizer`` under the reference's research path (``research/qwen2_5/qwen2_5_tokenizer.py``, also
``research/qwen2/qwen2_tokenizer.py``): byte-level BPE over ``vocab.json`` + ``merges.txt`` with the ChatML special tokens."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mindformers_b200.models.tokenizers import Qwen2Tokenizer  # noqa: E402,F401

Qwen2_5Tokenizer = Qwen2Tokenizer
__all__ = ["Qwen2Tokenizer", "Qwen2_5Tokenizer"]
