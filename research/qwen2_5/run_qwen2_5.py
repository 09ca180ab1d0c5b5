"""Qwen2.5 predict entry (reference ``research/qwen2_5/run_qwen2_5.py``): ``python research/qwen2_5/run_qwen2_5.py --config
configs/qwen2_5/predict_qwen2_5_7b.yaml --load_checkpoint <dir> --vocab_file vocab.json --merges_file merges.txt
--predict_data "..."``. Prompts are wrapped in the ChatML turn format the instruct checkpoints were tuned on."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from research.run_predict import main  # noqa: E402

SYSTEM = "You are a helpful assistant."


def chatml(prompt: str) -> str:
    return f"<|im_start|>system\n{SYSTEM}<|im_end|>\n<|im_start|>user\n{prompt}<|im_end|>\n<|im_start|>assistant\n"


if __name__ == "__main__":
    main(default_config=os.path.join(os.path.dirname(__file__), "..", "..", "configs", "qwen2_5", "predict_qwen2_5_7b.yaml"),
         wrap_prompt=chatml)
