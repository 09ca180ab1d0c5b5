from .causal_language_model_dataset import (BlendedMegatronDatasetDataLoader, CausalLanguageModelDataset,
                                            CommonDataLoader, GeneralDataset, IndexedDataLoader, KeyWordGenDataset,
                                            MockDataLoader, MultiTurnDataset, ResumableShardSampler, build_dataset,
                                            build_dataset_loader)
from .gpt_dataset import (BlendedDataset, BlendedMegatronDatasetBuilder, GPTDataset, GPTDatasetConfig, MockGPTDataset)
from .handlers import AlpacaInstructDataHandler, LlavaInstructDataHandler, PackingHandler, build_data_handler
from .modal_to_text_sft_dataset import ModalToTextSFTDataset
from .indexed_dataset import IndexedDataset, IndexedDatasetBuilder
from .dataloaders import (ADGenDataLoader, MultiSourceDataLoader, MultiSourceDataset, SFTDataLoader, ToolAlpacaDataLoader,
                          TrainingDataLoader, TrainingDataset, read_records)
from .sampler import build_sampler
from .transforms import build_transforms

from .._submodules import keep_functions as _keep_functions  # noqa: E402

_keep_functions(__name__, ('build_dataset',))
