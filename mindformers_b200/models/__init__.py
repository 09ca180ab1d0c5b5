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
                         PreTrainedTokenizerFast, Qwen2Tokenizer, TelechatTokenizer, convert_slow_tokenizer)


class BaseModel(PreTrainedModel):
    """Name of the reference's older model base class (``models/base_model.py:39``: a cell with the generation mixin,
    ``load_checkpoint`` from ``checkpoint_name_or_path`` in the configuration and the ``from_pretrained`` family).
    ``PreTrainedModel`` already is all of that; the alias keeps ``class MyModel(BaseModel)`` sources working and adds
    the ``load_checkpoint(config)`` entry point they call."""

    def load_checkpoint(self, config=None):
        path = getattr(config or self.model_config, "checkpoint_name_or_path", None)
        if not path:
            return None
        import os
        if os.path.isdir(path):
            return self.load_weights_from_dir(path)
        from ..checkpoint.io import load_checkpoint
        return load_checkpoint(path, self)


def build_model_config(config: dict = None, default_args=None, **kwargs):
    """Configuration object from the YAML ``model.model_config`` mapping (reference ``models/build_config.py``): ``type``
    names a registered configuration class; without it the class follows ``model_type`` / ``architectures``."""
    if config is None:
        return None
    if isinstance(config, PretrainedConfig):
        return config
    d = dict(config)
    if default_args:
        d.update(default_args)
    d.update(kwargs)
    name = d.pop("type", None)
    if name:
        from ..tools.register import MindFormerModuleType, MindFormerRegister
        if MindFormerRegister.is_exist(MindFormerModuleType.CONFIG, name):
            return MindFormerRegister.get_cls(MindFormerModuleType.CONFIG, name)(**d)
        import sys
        cls = getattr(sys.modules[__name__], name, None)
        if isinstance(cls, type) and issubclass(cls, PretrainedConfig):
            return cls(**d)
    from .auto import _classes_for
    return _classes_for(d)[0](**d)


def build_model(config: dict, default_args=None):
    """Older name of ``build_network`` (reference ``models/build_model.py``)."""
    return build_network(config, default_args)


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
