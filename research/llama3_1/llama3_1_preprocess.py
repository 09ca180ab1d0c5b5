"""Llama-3.1 dataset preprocessing entry (reference ``research/llama3_1/llama3_1_preprocess.py``): the command line of
``mindformers_b200/tools/dataset_preprocess/llama/llama_preprocess.py`` with the Llama-3 tokenizer as the default
(``--model_file`` is the tiktoken-style ``tokenizer.model``)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mindformers_b200.tools.dataset_preprocess.llama import llama_preprocess  # noqa: E402


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    if "--tokenizer" not in argv:
        argv += ["--tokenizer", "llama3"]
    return llama_preprocess.main(argv)


if __name__ == "__main__":
    main()
