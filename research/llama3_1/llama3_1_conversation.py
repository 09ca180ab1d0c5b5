"""Conversation templates under the reference's research path (``research/llama3_1/llama3_1_conversation.py``)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mindformers_b200.tools.dataset_preprocess.llama.conversation import *  # noqa: E402,F401,F403
