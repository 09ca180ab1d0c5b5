"""fp8 (e4m3, 128x128 block scales) → bf16 checkpoint cast under the reference's research path
(``research/deepseek3/fp8_cast_bf16.py``); the tool itself is ``toolkit/weight_convert/deepseekv3/fp8_cast_bf16.py``."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "toolkit", "weight_convert", "deepseekv3"))
from fp8_cast_bf16 import main  # noqa: E402

if __name__ == "__main__":
    main()
