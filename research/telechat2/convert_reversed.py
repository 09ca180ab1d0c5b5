"""Framework → Hugging Face weight conversion for this family (``research/telechat2/convert_reversed.py`` of the reference)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from convert_weight import main  # noqa: E402

if __name__ == "__main__":
    main(reversed_=True)
