"""Model families: configuration classes and ``…ForCausalLM`` classes, registered for YAML and Auto lookup.

Reference: ``models/llama`` (legacy), ``models/qwen2``, ``models/qwen3``, ``models/qwen3_moe``,
``models/deepseek3`` (mcore shims) and the research families (Llama-3.1, Qwen2.5, Mixtral, TeleChat2, GLM-4),
which here differ only in configuration defaults: all of them are instances of the same ``GPTModel``.
"""
from __future__ import annotations

from ..tools.register import MindFormerModuleType, MindFormerRegister
from .configuration_utils import PretrainedConfig
from .modeling_utils import PreTrainedModel

_BASE = dict(vocab_size=32000, hidden_size=4096, intermediate_size=11008, num_hidden_layers=32, num_attention_heads=32,
             num_key_value_heads=None, rms_norm_eps=1e-6, rope_theta=10000.0, max_position_embeddings=4096,
             tie_word_embeddings=False, pad_token_id=0, bos_token_id=1, eos_token_id=2)


def _config(name, model_type, defaults, is_mla=False):
    base = dict(_BASE)
    base.update(defaults)

    class _Cfg(PretrainedConfig):
        @classmethod
        def default_values(cls):
            return dict(base)

    _Cfg.__name__ = _Cfg.__qualname__ = name
    _Cfg.__doc__ = (f"Configuration of the ``{model_type}`` family with Hugging Face key names; defaults: "
                    + ", ".join(f"{k}={v!r}" for k, v in sorted(defaults.items())) + ".")
    _Cfg.model_type = model_type
    _Cfg.is_mla = is_mla
    MindFormerRegister.register_cls(_Cfg, MindFormerModuleType.CONFIG, alias=name)
    MindFormerRegister.register_cls(_Cfg, MindFormerModuleType.CONFIG, alias=name, legacy=False)
    return _Cfg


def _model(name, cfg_cls, family):
    class _M(PreTrainedModel):
        config_class = cfg_cls
        weight_family = family

    _M.__name__ = _M.__qualname__ = name
    _M.__doc__ = (f"Causal language model of the ``{family}`` family: ``{cfg_cls.__name__}`` → ``GPTModel``; Hugging Face "
                  f"checkpoints are mapped by the ``{family}`` name rules (``checkpoint/name_maps.py``).")
    MindFormerRegister.register_cls(_M, MindFormerModuleType.MODELS, alias=name)
    MindFormerRegister.register_cls(_M, MindFormerModuleType.MODELS, alias=name, legacy=False)
    return _M


LlamaConfig = _config("LlamaConfig", "llama", dict(rms_norm_eps=1e-5))
Qwen2Config = _config("Qwen2Config", "qwen2", dict(vocab_size=152064, attention_bias=True, rope_theta=1e6))
Qwen3Config = _config("Qwen3Config", "qwen3", dict(vocab_size=151936, qk_layernorm=True, head_dim=128, rope_theta=1e6))
Qwen3MoeConfig = _config("Qwen3MoeConfig", "qwen3_moe",
                         dict(vocab_size=151936, qk_layernorm=True, head_dim=128, rope_theta=1e6, num_experts=128,
                              num_experts_per_tok=8, moe_intermediate_size=768, norm_topk_prob=True,
                              first_k_dense_replace=0, moe_router_score_function="softmax"))
DeepseekV3Config = _config("DeepseekV3Config", "deepseek_v3",
                           dict(vocab_size=129280, hidden_size=7168, intermediate_size=18432, num_hidden_layers=61,
                                num_attention_heads=128, num_key_value_heads=128, n_routed_experts=256,
                                n_shared_experts=1, num_experts_per_tok=8, moe_intermediate_size=2048, n_group=8,
                                topk_group=4, routed_scaling_factor=2.5, norm_topk_prob=True, scoring_func="sigmoid",
                                first_k_dense_replace=3, q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128,
                                qk_rope_head_dim=64, v_head_dim=128, moe_router_enable_expert_bias=True,
                                rope_interleave=True), is_mla=True)
DeepseekV2Config = _config("DeepseekV2Config", "deepseek_v2",
                           dict(vocab_size=102400, hidden_size=5120, intermediate_size=12288, num_hidden_layers=60,
                                num_attention_heads=128, num_key_value_heads=128, n_routed_experts=160,
                                n_shared_experts=2, num_experts_per_tok=6, moe_intermediate_size=1536, n_group=8,
                                topk_group=3, routed_scaling_factor=16.0, norm_topk_prob=False, scoring_func="softmax",
                                first_k_dense_replace=1, q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128,
                                qk_rope_head_dim=64, v_head_dim=128, rope_interleave=True), is_mla=True)
Qwen2MoeConfig = _config("Qwen2MoeConfig", "qwen2_moe",
                         dict(vocab_size=151936, attention_bias=True, rope_theta=1e6, num_experts=60,
                              num_experts_per_tok=4, moe_intermediate_size=1408, shared_expert_intermediate_size=5632,
                              use_shared_expert_gating=True, norm_topk_prob=False, first_k_dense_replace=0,
                              moe_router_score_function="softmax"))
MixtralConfig = _config("MixtralConfig", "mixtral",
                        dict(num_experts=8, num_experts_per_tok=2, moe_intermediate_size=14336, norm_topk_prob=True,
                             first_k_dense_replace=0, num_key_value_heads=8, rope_theta=1e6))
TelechatConfig = _config("TelechatConfig", "telechat", dict(vocab_size=131072))


class ChatGLM2Config(PretrainedConfig):
    """ChatGLM2 / ChatGLM3 / GLM-4 configuration with the keys of the reference's class and of the published
    ``config.json`` files (``models/glm2/glm2_config.py:125-240``: ``padded_vocab_size``, ``num_layers``,
    ``ffn_hidden_size``, ``kv_channels``, ``multi_query_attention`` / ``multi_query_group_num``, ``rope_ratio``,
    ``rmsnorm``, ``add_qkv_bias`` …); defaults are GLM-4-9B.

    What makes the family differ from Llama is expressed in ``to_transformer_dict``: the rotary embedding covers the
    first half of every head and rotates adjacent pairs (``glm2_modules.py`` rotary: ``rope_cache`` over
    ``kv_channels // 2`` dims, pairs ``(2i, 2i+1)``), its base is ``10000 * rope_ratio``, Q/K/V carry a bias while the
    other projections do not, and there are ``multi_query_group_num`` KV heads."""

    model_type = "glm"

    @classmethod
    def default_values(cls):
        return dict(num_layers=40, padded_vocab_size=151552, hidden_size=4096, ffn_hidden_size=13696, kv_channels=128,
                    num_attention_heads=32, seq_length=8192, layernorm_epsilon=1.5625e-07, rope_ratio=1.0, rmsnorm=True,
                    post_layer_norm=True, add_bias_linear=False, add_qkv_bias=True, multi_query_attention=True,
                    multi_query_group_num=2, tie_word_embeddings=False, pad_token_id=151329, eos_token_id=151329,
                    max_position_embeddings=None)

    _PAIRS = (("num_layers", "num_hidden_layers"), ("padded_vocab_size", "vocab_size"),
              ("ffn_hidden_size", "intermediate_size"), ("kv_channels", "head_dim"),
              ("multi_query_group_num", "num_key_value_heads"), ("layernorm_epsilon", "rms_norm_eps"),
              ("add_qkv_bias", "attention_bias"), ("rope_ratio", "rope_theta"), ("rope_ratio", "rotary_base"))

    def __init__(self, **kwargs):
        self._explicit = set(kwargs)
        super().__init__(**kwargs)

    def to_transformer_dict(self) -> dict:
        d = self.to_dict()
        # a configuration written with Hugging Face keys (the GLM-4-0414 ``config.json`` spelling) wins over this
        # class's ChatGLM-keyed defaults
        for glm_key, hf_key in self._PAIRS:
            if d.get(hf_key) is not None and glm_key not in self._explicit:
                d.pop(glm_key, None)
        if "rope_ratio" not in d:
            d.pop("multi_query_attention", None)
            if "partial_rotary_factor" not in d:
                d.setdefault("rotary_percent", 0.5)
            d.setdefault("rotary_interleaved", True)
            d["normalization"] = "RMSNorm" if d.pop("rmsnorm", True) else "LayerNorm"
            return d
        if not d.pop("multi_query_attention", True):
            d["multi_query_group_num"] = d["num_attention_heads"]
        d["rotary_base"] = 10000.0 * float(d.pop("rope_ratio", 1.0) or 1.0)
        d.setdefault("rotary_percent", 0.5)
        d.setdefault("rotary_interleaved", True)
        d["normalization"] = "RMSNorm" if d.pop("rmsnorm", True) else "LayerNorm"
        if d.get("max_position_embeddings") is None:
            d["max_position_embeddings"] = d.get("seq_length")
        if "vocab_size" in d and "padded_vocab_size" in d:
            d.pop("vocab_size")
        return d


MindFormerRegister.register_cls(ChatGLM2Config, MindFormerModuleType.CONFIG, alias="ChatGLM2Config")
MindFormerRegister.register_cls(ChatGLM2Config, MindFormerModuleType.CONFIG, alias="ChatGLM2Config", legacy=False)
ChatGLM4Config = ChatGLM2Config

LlamaForCausalLM = _model("LlamaForCausalLM", LlamaConfig, "llama")
Qwen2ForCausalLM = _model("Qwen2ForCausalLM", Qwen2Config, "qwen2")
Qwen3ForCausalLM = _model("Qwen3ForCausalLM", Qwen3Config, "qwen3")
Qwen3MoeForCausalLM = _model("Qwen3MoeForCausalLM", Qwen3MoeConfig, "qwen3_moe")
DeepseekV3ForCausalLM = _model("DeepseekV3ForCausalLM", DeepseekV3Config, "deepseek_v3")
DeepseekV2ForCausalLM = _model("DeepseekV2ForCausalLM", DeepseekV2Config, "deepseek_v2")
Qwen2MoeForCausalLM = _model("Qwen2MoeForCausalLM", Qwen2MoeConfig, "qwen2_moe")
MixtralForCausalLM = _model("MixtralForCausalLM", MixtralConfig, "mixtral")
TelechatForCausalLM = _model("TelechatForCausalLM", TelechatConfig, "telechat")
ChatGLM2ForConditionalGeneration = _model("ChatGLM2ForConditionalGeneration", ChatGLM4Config, "glm")

def _backbone(name, causal_cls):
    class _B(causal_cls):
        def forward(self, input_ids, position_ids=None, attn_meta=None, **kw):
            return self.model(input_ids, None, None, position_ids, attn_meta, return_hidden=True,
                              input_embeds=kw.get("input_embeds"))

    _B.__name__ = _B.__qualname__ = name
    _B.__doc__ = (f"The ``{causal_cls.__name__}`` network without its language-model head: ``forward(input_ids)`` returns the "
                  f"final-norm hidden states ``[B * S, hidden]`` (reference ``models/llama/llama.py`` ``LlamaModel``, "
                  f"``models/glm2/glm2.py`` ``ChatGLM2Model``). The head's weights are still built so that a causal-LM "
                  f"checkpoint loads without missing keys.")
    return _B


LlamaModel = _backbone("LlamaModel", LlamaForCausalLM)
ChatGLM2Model = _backbone("ChatGLM2Model", ChatGLM2ForConditionalGeneration)


class ChatGLM2WithPtuning2(ChatGLM2ForConditionalGeneration):
    """ChatGLM2 with P-Tuning v2 (reference ``models/glm2/glm2.py`` ``ChatGLM2WithPtuning2``): the base weights are frozen
    and a per-layer key / value prefix of ``config.pet_config.pre_seq_len`` virtual tokens is trained."""

    def __init__(self, config, **kwargs):
        super().__init__(config, **kwargs)
        from ..pet.pet_config import Ptuning2Config
        from ..pet.prompt import PrefixTuningModel
        pet = getattr(config, "pet_config", None) or {}
        if not isinstance(pet, Ptuning2Config):
            pet = dict(pet)
            pet.pop("pet_type", None)
            pet = Ptuning2Config(**pet)
        tuned = PrefixTuningModel(pet, self)
        object.__setattr__(self, "_tuned", tuned)           # not a sub-module: it holds this module already
        self.prefix_encoder = tuned.prefix_encoder

    def forward(self, *args, **kwargs):
        self._tuned.current = self.prefix_encoder()
        return super().forward(*args, **kwargs)


# Names that configurations written for the reference use for the same models: its mcore shims pick a
# ``Training...`` or ``Inference...`` class by run mode (``qwen3/modeling_qwen3.py:27-54``,
# ``deepseek3/modeling_deepseek_v3.py:25-42``) and its research directories ship explicit tensor-parallel inference
# models (``research/llama3_1/llama.py:48`` ``ParallelLlamaForCausalLM``, ``research/qwen2_5`` ``ParallelQwenForCausalLM``,
# ``research/deepseek3`` ``DeepseekV3ForCausalLM`` / ``InferenceDeepseekV3ForCausalLM``). One class serves training and
# inference here, so these are aliases.
_ALIASES = {
    "ParallelLlamaForCausalLM": LlamaForCausalLM, "ParallelQwenForCausalLM": Qwen2ForCausalLM,
    "TrainingQwen3ForCausalLM": Qwen3ForCausalLM, "InferenceQwen3ForCausalLM": Qwen3ForCausalLM,
    "TrainingQwen3MoeForCausalLM": Qwen3MoeForCausalLM, "InferenceQwen3MoeForCausalLM": Qwen3MoeForCausalLM,
    "TrainingDeepseekV3ForCausalLM": DeepseekV3ForCausalLM, "InferenceDeepseekV3ForCausalLM": DeepseekV3ForCausalLM,
    "InferenceQwen2ForCausalLM": Qwen2ForCausalLM, "DeepseekV2ForCausalLM_legacy": DeepseekV2ForCausalLM,
    "TelechatForCausalLM_MoE": TelechatForCausalLM,
}
globals().update(_ALIASES)
for _alias, _cls in _ALIASES.items():
    for _legacy in (True, False):
        MindFormerRegister.register_cls(_cls, MindFormerModuleType.MODELS, alias=_alias, legacy=_legacy)

MODEL_TYPE_TO_CLASSES = {
    "llama": (LlamaConfig, LlamaForCausalLM), "qwen2": (Qwen2Config, Qwen2ForCausalLM),
    "qwen2_5": (Qwen2Config, Qwen2ForCausalLM), "qwen3": (Qwen3Config, Qwen3ForCausalLM),
    "qwen3_moe": (Qwen3MoeConfig, Qwen3MoeForCausalLM), "deepseek_v3": (DeepseekV3Config, DeepseekV3ForCausalLM),
    "deepseekv3": (DeepseekV3Config, DeepseekV3ForCausalLM), "mixtral": (MixtralConfig, MixtralForCausalLM),
    "deepseek_v2": (DeepseekV2Config, DeepseekV2ForCausalLM), "deepseek2": (DeepseekV2Config, DeepseekV2ForCausalLM),
    "qwen2_moe": (Qwen2MoeConfig, Qwen2MoeForCausalLM),
    "telechat": (TelechatConfig, TelechatForCausalLM), "glm": (ChatGLM4Config, ChatGLM2ForConditionalGeneration),
    "chatglm": (ChatGLM4Config, ChatGLM2ForConditionalGeneration),
}
