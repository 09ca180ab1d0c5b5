"""Processor bases (reference ``models/base_processor.py``: ``BaseAudioProcessor:32``, ``BaseProcessor``)."""
from ..models.processing_utils import BaseProcessor  # noqa: F401
from ..models.multi_modal import BaseImageProcessor  # noqa: F401


class BaseAudioProcessor:
    """Base of audio pre-processors: keeps its keyword arguments in ``config``; calling it runs ``preprocess(audio_data)``,
    which every audio processor implements (the feature extraction helpers are in ``dataset/transforms/audio_utils.py``)."""

    def __init__(self, **kwargs):
        self.config = dict(kwargs)

    def __call__(self, audio_data, **kwargs):
        return self.preprocess(audio_data, **kwargs)

    def preprocess(self, audio_data, **kwargs):
        raise NotImplementedError("every audio processor implements its own preprocess method")


__all__ = ["BaseAudioProcessor", "BaseImageProcessor", "BaseProcessor"]
