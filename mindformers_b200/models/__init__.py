from .auto import AutoConfig, AutoModel, AutoModelForCausalLM, AutoProcessor, AutoTokenizer
from .configuration_utils import PretrainedConfig
from .families import (ChatGLM2ForConditionalGeneration, DeepseekV2Config, DeepseekV2ForCausalLM, DeepseekV3Config,
                       DeepseekV3ForCausalLM, LlamaConfig, Qwen2MoeConfig, Qwen2MoeForCausalLM,
                       LlamaForCausalLM, MixtralConfig, MixtralForCausalLM, Qwen2Config, Qwen2ForCausalLM, Qwen3Config,
                       Qwen3ForCausalLM, Qwen3MoeConfig, Qwen3MoeForCausalLM, TelechatConfig, TelechatForCausalLM)
from .families import ChatGLM2Config
from .modeling_utils import PreTrainedModel
from .llama_legacy import LegacyLlamaForCausalLM, LlamaLegacyConfig
from .presets import PRESETS, get_preset
from .tokenization import ByteTokenizer, TextProcessor, build_tokenizer
from .tokenization_utils import AddedToken, BatchEncoding, BytePairEncoder, PreTrainedTokenizer
from .tokenizers import (ChatGLM3Tokenizer, ChatGLM4Tokenizer, Llama3Tokenizer, LlamaTokenizer, LlamaTokenizerFast,
                         Qwen2Tokenizer, TelechatTokenizer)


def build_network(config: dict, default_args=None):
    """Model from the YAML ``model`` section: ``{"arch": {"type": ...}, "model_config": {...}}``."""
    mc = dict(config.get("model_config") or {})
    if default_args:
        mc.update(default_args)
    arch = (config.get("arch") or {}).get("type")
    if arch and "architectures" not in mc:
        mc["architectures"] = [arch]
    mc.pop("type", None)
    return AutoModel.from_config(mc)
from .processing_utils import BaseProcessor, GLMProcessor, LlamaProcessor, ProcessorMixin, build_processor
