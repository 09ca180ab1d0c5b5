"""Alpaca JSON → conversation-format JSON (reference ``research/qwen2/alpaca_converter.py``); the converter itself is
``mindformers_b200/tools/dataset_preprocess/llama/alpaca_converter.py``."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mindformers_b200.tools.dataset_preprocess.llama.alpaca_converter import main  # noqa: E402

if __name__ == "__main__":
    main()
