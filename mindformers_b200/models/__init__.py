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


# keys of the older top-level ``moe_config`` YAML section that steer MindSpore's MoE implementation only (routing class
# names, graph-fusion switches, drop-rate callbacks): nothing to translate
_MOE_LEGACY_ONLY = {"routing_policy", "enable_sdrop", "use_fused_ops_topkrouter", "use_fused_ops_permute", "group_wise_a2a",
                    "comp_comm_parallel", "comp_comm_parallel_degree", "ep_extend_tp", "callback_moe_droprate",
                    "save_token_distribution", "cur_layer", "enable_cold_hot_expert", "hot_expert_num", "cold_token_percent",
                    "moe_module_name", "enable_gmm_safe_tokens", "use_3d_tensor_parallel", "tp_x", "tp_y", "tp_z",
                    "moe_shared_expert_overlap", "use_shared_expert_gating", "max_router_load", "expert_group_size",
                    "enable_delay_allreduce"}


def merge_moe_config(model_config: dict, moe_config) -> dict:
    """Fold the older ``moe_config`` section (reference ``modules/transformer/moe.py:88`` ``MoEConfig``; top level of the
    legacy YAMLs, e.g. ``research/telechat2/telechat2-39b-a12b/finetune_telechat_39b_a12b.yaml:34-50``) into the model
    configuration: ``expert_num`` / ``num_experts_chosen`` / ``capacity_factor`` / ... are aliases the configuration
    converter knows; ``aux_loss_factors`` + ``aux_loss_types`` become the one load-balancing coefficient; keys that only
    select MindSpore code paths are dropped. Keys already present in the model configuration win."""
    if not moe_config:
        return model_config
    moe = dict(moe_config.to_dict() if hasattr(moe_config, "to_dict") and not isinstance(moe_config, dict) else moe_config)
    out = dict(model_config)
    factors, types = moe.pop("aux_loss_factors", None), moe.pop("aux_loss_types", None)
    if factors:
        types = list(types or ["expert"] * len(factors))
        coeff = next((f for f, t in zip(factors, types) if t == "expert"), factors[0])
        if coeff:
            moe.setdefault("router_aux_loss_coef", coeff)
    if int(moe.get("expert_num", 1) or 1) <= 1:
        return out                                        # a dense model that carries the section's defaults
    if moe.get("shared_expert_num") in (0, None):
        moe.pop("shared_expert_num", None)
    moe.pop("capacity_factor", None)                      # the expert layers here are dropless: no token is cut off
    for k, v in moe.items():
        if k in _MOE_LEGACY_ONLY or v is None:
            continue
        out.setdefault(k, v)
    return out


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
    mc = merge_moe_config(mc, mc.pop("moe_config", None) or config.get("moe_config"))
    arch = (config.get("arch") or {}).get("type")
    if arch and "architectures" not in mc:
        mc["architectures"] = [arch]
    mc.pop("type", None)
    return AutoModel.from_config(mc)
from .processing_utils import BaseProcessor, GLMProcessor, LlamaProcessor, ProcessorMixin, build_processor

from .._submodules import keep_functions as _keep_functions  # noqa: E402

_keep_functions(__name__, ('build_model', 'build_processor', 'build_tokenizer', 'convert_slow_tokenizer'))
