"""Tensor layout helpers of the weight converters (reference ``utils/convert_utils.py``: q/k/v and gate/up concatenation)."""
from ..checkpoint.name_maps import fuse_state_dict, hf_to_framework, framework_to_hf  # noqa: F401

__all__ = ["framework_to_hf", "fuse_state_dict", "hf_to_framework"]
