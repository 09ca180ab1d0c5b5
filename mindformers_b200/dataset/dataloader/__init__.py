"""Data loaders under the reference's ``dataset/dataloader`` path."""
from ...dataset.dataloaders import ADGenDataLoader, BaseMultiModalDataLoader, HFDataLoader, MultiModalSFTDataLoader, MultiSourceDataLoader, SFTDataLoader, ToolAlpacaDataLoader, TrainingDataLoader  # noqa: F401
from ...dataset.causal_language_model_dataset import BlendedMegatronDatasetDataLoader, CommonDataLoader, IndexedDataLoader, build_dataset_loader  # noqa: F401

__all__ = ["ADGenDataLoader", "BaseMultiModalDataLoader", "BlendedMegatronDatasetDataLoader", "CommonDataLoader", "HFDataLoader", "IndexedDataLoader", "MultiModalSFTDataLoader", "MultiSourceDataLoader", "SFTDataLoader", "ToolAlpacaDataLoader", "TrainingDataLoader", "build_dataset_loader"]
