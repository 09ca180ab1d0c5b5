"""Megatron-style blended datasets under the reference's ``dataset/blended_datasets`` path."""
from ...dataset.gpt_dataset import BlendedDataset, BlendedMegatronDatasetBuilder, GPTDataset, GPTDatasetConfig, MockGPTDataset  # noqa: F401
from ...dataset.indexed_dataset import IndexedDataset, IndexedDatasetBuilder  # noqa: F401

__all__ = ["BlendedDataset", "BlendedMegatronDatasetBuilder", "GPTDataset", "GPTDatasetConfig", "IndexedDataset", "IndexedDatasetBuilder", "MockGPTDataset"]
