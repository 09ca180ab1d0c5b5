"""``Llama3Tokenizer`` under the reference's research path (``research/llama3_1/llama3_1_tokenizer.py``): the tiktoken-style
byte-pair tokenizer of Llama 3 / 3.1 (``tokenizer.model`` with base64 ranks, 256 reserved special tokens)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mindformers_b200.models.tokenizers import Llama3Tokenizer  # noqa: E402,F401

__all__ = ["Llama3Tokenizer"]
