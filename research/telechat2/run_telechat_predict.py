"""TeleChat2 predict entry (reference ``research/telechat2/run_telechat_predict.py``): ``--yaml_file``, ``--checkpoint_path``,
``--vocab_file_path``, ``--max_new_tokens`` ...; prompts are wrapped in TeleChat's ``<_user>...<_bot>`` turn format."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from research.run_predict import main  # noqa: E402


def telechat_turn(prompt: str) -> str:
    return f"<_user>{prompt}<_bot>"


if __name__ == "__main__":
    main(wrap_prompt=telechat_turn)
