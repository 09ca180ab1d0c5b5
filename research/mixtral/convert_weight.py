"""Hugging Face → framework weight conversion for this family under the reference's research path
(``research/mixtral/convert_weight.py``): ``python research/mixtral/convert_weight.py --input_path <hf dir> --output_path <out>``
is ``python convert_weight.py --model mixtral ...``; ``convert_reversed.py`` beside it adds ``--reversed``."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import convert_weight  # noqa: E402


def main(argv=None, reversed_=False):
    argv = list(sys.argv[1:] if argv is None else argv)
    if "--model" not in argv:
        argv = ["--model", "mixtral"] + argv
    if reversed_ and "--reversed" not in argv:
        argv.append("--reversed")
    return convert_weight.main(argv)


if __name__ == "__main__":
    main()
