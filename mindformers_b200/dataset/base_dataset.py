"""Shard bookkeeping of the datasets (reference ``dataset/base_dataset.py:66-107``)."""
from ..dataset.causal_language_model_dataset import data_shard_info, ResumableShardSampler  # noqa: F401

__all__ = ["ResumableShardSampler", "data_shard_info"]
