"""``ParallelLlamaForCausalLM`` (reference ``research/llama3_1/llama.py:48``): the reference keeps a separate explicitly
tensor-parallel inference network; here ``LlamaForCausalLM`` shards itself over the tensor-parallel group that
``parallel_state`` holds, so the name is an alias (it is also registered under this name for ``model.arch.type``)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mindformers_b200.models.families import LlamaForCausalLM as ParallelLlamaForCausalLM  # noqa: E402,F401

__all__ = ["ParallelLlamaForCausalLM"]
