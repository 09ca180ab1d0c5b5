from .beam_search import BeamSearchScorer
from .generation_config import GenerationConfig
from .logits_process import (FrequencyPenaltyLogitsProcessor, LogitNormalization, LogitsProcessor, LogitsProcessorList,
                             MinLengthLogitsProcessor, MinNewTokensLengthLogitsProcessor,
                             PresencePenaltyLogitsProcessor, RepetitionPenaltyLogitsProcessor, SamplingLogitsProcessor,
                             TemperatureLogitsWarper, TopKLogitsWarper, TopPLogitsWarper)
from .streamers import BaseStreamer, TextIteratorStreamer, TextStreamer
from .text_generator import GenerationMixin
