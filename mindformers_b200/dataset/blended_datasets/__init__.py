"""Megatron-style blended datasets under the reference's ``dataset/blended_datasets`` path."""
from ...dataset.gpt_dataset import (BlendedDataset, BlendedMegatronDatasetBuilder, BlendedMegatronDatasetConfig, GPTDataset,  # noqa: F401
                                    GPTDatasetConfig, MockGPTDataset, Split, convert_split_vector_to_split_matrix,
                                    get_blend_from_list, normalize, parse_and_normalize_split)
from ...dataset.helpers import (build_blending_indices, build_exhaustive_blending_indices, build_sample_idx,  # noqa: F401
                                compile_helpers)
from ...dataset.indexed_dataset import IndexedDataset, IndexedDatasetBuilder  # noqa: F401

MegatronDataset = GPTDataset

__all__ = ["BlendedDataset", "BlendedMegatronDatasetBuilder", "BlendedMegatronDatasetConfig", "GPTDataset", "GPTDatasetConfig",
           "IndexedDataset", "IndexedDatasetBuilder", "MegatronDataset", "MockGPTDataset", "Split", "build_blending_indices",
           "build_exhaustive_blending_indices", "build_sample_idx", "compile_helpers", "convert_split_vector_to_split_matrix",
           "get_blend_from_list", "normalize", "parse_and_normalize_split"]
