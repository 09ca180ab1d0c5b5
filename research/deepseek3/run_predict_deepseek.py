"""DeepSeek-V3 / R1 predict entry (reference ``research/deepseek3/run_predict_deepseek.py``): ``--config`` a predict YAML
(``configs/deepseek3/predict_deepseek3_671b.yaml`` or the W8A8 one), ``--input`` the prompt(s). Launch one process per
GPU with ``scripts/launcher.sh`` for the tensor- / expert-parallel layouts those YAMLs describe."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from research.run_predict import main  # noqa: E402


def deepseek_chat(prompt: str) -> str:
    return f"<｜begin▁of▁sentence｜><｜User｜>{prompt}<｜Assistant｜>"


if __name__ == "__main__":
    main(default_config=os.path.join(os.path.dirname(__file__), "..", "..", "configs", "deepseek3", "predict_deepseek3_671b.yaml"),
         default_prompt="生抽与老抽的区别？", wrap_prompt=deepseek_chat)
