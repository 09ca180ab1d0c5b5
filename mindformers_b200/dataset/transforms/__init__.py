"""Image and audio transforms of the multimodal datasets (reference ``mindformers/dataset/transforms``)."""
from .audio_utils import (amplitude_to_db, hertz_to_mel, mel_filter_bank, mel_to_hertz, optimal_fft_length, power_to_db,
                          spectrogram, window_function)
from .build_transforms import Compose, build_transforms
from .vision_transforms import (BCHW2BHWC, BatchCenterCrop, BatchNormalize, BatchPILize, BatchResize, BatchToTensor,
                                RandomCropDecodeResize, RandomHorizontalFlip, RandomResizedCrop, Resize)

__all__ = ["BCHW2BHWC", "BatchCenterCrop", "BatchNormalize", "BatchPILize", "BatchResize", "BatchToTensor", "Compose",
           "RandomCropDecodeResize", "RandomHorizontalFlip", "RandomResizedCrop", "Resize", "amplitude_to_db",
           "build_transforms", "hertz_to_mel", "mel_filter_bank", "mel_to_hertz", "optimal_fft_length", "power_to_db",
           "spectrogram", "window_function"]

from ..._submodules import keep_functions as _keep_functions  # noqa: E402

_keep_functions(__name__, ('build_transforms',))
