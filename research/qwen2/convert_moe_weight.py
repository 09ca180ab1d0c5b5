"""Qwen1.5 / Qwen2 MoE weight conversion (reference ``research/qwen2/convert_moe_weight.py``):
``python convert_weight.py --model qwen2_moe ...``."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import convert_weight  # noqa: E402

if __name__ == "__main__":
    argv = sys.argv[1:]
    convert_weight.main(argv if "--model" in argv else ["--model", "qwen2_moe"] + argv)
