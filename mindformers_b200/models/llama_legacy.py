"""The ``use_legacy: True`` Llama: reference configuration keys and reference parameter names.

The reference keeps a pre-mcore Llama implementation (``models/llama/llama.py:55-420`` ``LlamaModel`` /
``LlamaForCausalLM``, ``llama_transformer.py`` ``LLamaAttention`` / ``LLamaDecodeLayer``, ``llama_layer.py``
``LlamaFeedForward`` / ``LlamaEmbedding``) whose checkpoints name their tensors
``model.tok_embeddings.embedding_weight``, ``model.layers.N.attention.{wq,wk,wv,wo}.weight`` (``w_qkv`` with
``qkv_concat``), ``model.layers.N.feed_forward.{w1,w2,w3}.weight`` (``w_gate_hidden`` with ``qkv_concat``),
``model.layers.N.{attention_norm,ffn_norm}.weight``, ``model.norm_out.weight`` and ``lm_head.weight``, and whose
configuration sizes the feed-forward from ``multiple_of`` / ``ffn_dim_multiplier`` when ``intermediate_size`` is
absent (``llama_layer.py:305-320``).

Here the arithmetic is that of ``GPTModel`` (one fused QKV GEMM, one fused gate/up GEMM); the class keeps the legacy
*interface*: it is built from the legacy keys, ``state_dict()`` / ``parameters_dict()`` emit the legacy names (views
of the fused parameters, so nothing is copied) and ``load_state_dict()`` / ``load_weights()`` take them.
"""
from __future__ import annotations

from typing import Dict, Iterator, Tuple

import torch

from ..checkpoint import name_maps
from ..tools.register import MindFormerModuleType, MindFormerRegister
from .configuration_utils import PretrainedConfig
from .modeling_utils import PreTrainedModel


def legacy_ffn_hidden_size(hidden_size: int, intermediate_size=None, multiple_of: int = 256, ffn_dim_multiplier=None) -> int:
    """Width of the gated feed-forward as the legacy ``LlamaFeedForward`` derives it."""
    if intermediate_size:
        return int(intermediate_size)
    dim = int(2 * (4 * hidden_size) / 3)
    if ffn_dim_multiplier is not None:
        dim = int((ffn_dim_multiplier + 0.01) * dim)
    return multiple_of * ((dim + multiple_of - 1) // multiple_of)


class LlamaLegacyConfig(PretrainedConfig):
    """Legacy Llama configuration (``models/llama/llama_config.py:40-200``): ``num_layers``, ``num_heads``,
    ``n_kv_heads``, ``hidden_size``, ``intermediate_size`` or ``multiple_of`` + ``ffn_dim_multiplier``, ``rms_norm_eps``,
    ``theta``, ``seq_length``, ``vocab_size``, ``qkv_concat``, ``scaling_factor`` / ``extend_method``."""

    model_type = "llama"

    @classmethod
    def default_values(cls):
        return dict(batch_size=1, seq_length=2048, hidden_size=4096, num_layers=32, num_heads=32, n_kv_heads=None,
                    vocab_size=32000, intermediate_size=None, multiple_of=256, ffn_dim_multiplier=None,
                    rms_norm_eps=1e-5, theta=10000.0, qkv_concat=False, tie_word_embeddings=False, pad_token_id=0,
                    bos_token_id=1, eos_token_id=2, max_position_embeddings=None)

    def to_transformer_dict(self) -> dict:
        d = self.to_dict()
        # a configuration written with Hugging Face keys wins over this class's legacy-keyed defaults
        for legacy, hf in (("num_layers", "num_hidden_layers"), ("num_heads", "num_attention_heads"),
                           ("n_kv_heads", "num_key_value_heads"), ("theta", "rope_theta"),
                           ("rms_norm_eps", "layernorm_epsilon"), ("intermediate_size", "ffn_hidden_size")):
            if d.get(hf) is not None:
                d.pop(legacy, None)
        if d.get("ffn_hidden_size") is not None:
            d.pop("multiple_of", None), d.pop("ffn_dim_multiplier", None)
            return self._finish(d)
        d["intermediate_size"] = legacy_ffn_hidden_size(d["hidden_size"], d.get("intermediate_size"),
                                                        d.pop("multiple_of", 256) or 256, d.pop("ffn_dim_multiplier", None))
        return self._finish(d)

    @staticmethod
    def _finish(d: dict) -> dict:
        if "n_kv_heads" in d and d["n_kv_heads"] is None:
            d["n_kv_heads"] = d.get("num_heads") or d.get("num_attention_heads")
        if d.get("max_position_embeddings") is None:
            d["max_position_embeddings"] = d["seq_length"]
        return d


class LegacyLlamaForCausalLM(PreTrainedModel):
    """Llama with the reference's legacy parameter names on the outside (``models/llama/llama.py:423-702``)."""

    config_class = LlamaLegacyConfig
    weight_family = "llama"

    def _qkv_concat(self) -> bool:
        return bool(getattr(self.model_config, "qkv_concat", False))

    # ---- legacy names out ---------------------------------------------------------------------------------
    def legacy_named_parameters(self) -> Iterator[Tuple[str, torch.Tensor]]:
        """``(legacy name, tensor)`` for every parameter: slices of ``linear_qkv`` as ``wq / wk / wv`` and halves of
        ``linear_fc1`` as ``w1 / w3`` (or the fused tensors as ``w_qkv`` / ``w_gate_hidden`` with ``qkv_concat``). The
        tensors are views: writing through them updates the model."""
        own = {n: p.detach() for n, p in self.named_parameters()}
        yield from name_maps.framework_to_legacy_llama(own, self.config, self._qkv_concat()).items()

    def parameters_dict(self) -> Dict[str, torch.Tensor]:
        return dict(self.legacy_named_parameters())

    def state_dict(self, *args, **kwargs):          # noqa: D401 - torch signature
        return self.parameters_dict()

    # ---- legacy names in ----------------------------------------------------------------------------------
    def load_state_dict(self, state_dict, strict: bool = True, assign: bool = False):
        """Accepts legacy names, Hugging Face names or this framework's own names."""
        keys = list(state_dict)
        if any(name_maps.is_legacy_llama_name(k) for k in keys):
            state_dict = name_maps.legacy_llama_to_framework(state_dict, self.config)
        elif any(k.startswith(("model.embed_tokens", "model.layers.")) and ".self_attn." in k or k.startswith("lm_head")
                 for k in keys):
            state_dict = name_maps.hf_to_framework(state_dict, self.config, "llama")
        return self.model.load_state_dict(state_dict, strict=strict)

    @classmethod
    def convert_name(cls, weight_name: str) -> str:           # Hugging Face name -> legacy name, as the reference's hook
        return name_maps.convert_name_legacy(weight_name)


for _legacy in (True, False):
    MindFormerRegister.register_cls(LlamaLegacyConfig, MindFormerModuleType.CONFIG, alias="LlamaLegacyConfig", legacy=_legacy)
    MindFormerRegister.register_cls(LegacyLlamaForCausalLM, MindFormerModuleType.MODELS, alias="LegacyLlamaForCausalLM",
                                    legacy=_legacy)
