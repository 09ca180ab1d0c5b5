"""``PreTrainedModel``: base of every causal-LM class (build, load, save, generate).

Reference: ``models/modeling_utils.py`` (``PreTrainedModel`` :216, ``from_pretrained`` :855-1266,
``save_pretrained`` with sharding :87, name-conversion hooks :1507-1522) and the per-model shims
(``qwen3/modeling_qwen3.py:27-54`` etc.). Unlike the reference there is one network class for training and
inference; ``RUN_MODE=predict`` only changes defaults (eval mode, no optimizer).
"""
from __future__ import annotations

import json
import os
from typing import Optional

import torch
import torch.nn as nn

from ..checkpoint import io as ckpt_io
from ..checkpoint import name_maps
from ..generation import GenerationConfig, GenerationMixin
from ..inference.model_utils import InferModelMixin
from ..parallel.layers.gpt_model import GPTModel
from ..parallel.transformer_config_utils import convert_to_transformer_config
from ..tools.logger import logger
from .configuration_utils import PretrainedConfig


class PreTrainedModel(nn.Module, GenerationMixin, InferModelMixin):
    """Base of the model classes (reference ``models/modeling_utils.py:216``): holds the Hugging Face keyed
    ``config``, builds the ``GPTModel`` from it, and provides ``from_pretrained`` / ``save_pretrained`` (sharded
    safetensors + ``config.json``), the name-conversion hooks (``convert_name``, ``convert_weight_dict``,
    ``obtain_name_map``), ``generate()`` (``GenerationMixin``) and the serving helpers of ``InferModelMixin``."""

    config_class = PretrainedConfig
    base_model_prefix = "model"
    weight_family = "llama"

    def __init__(self, config: PretrainedConfig, device=None, dtype=None, **kwargs):
        super().__init__()
        if isinstance(config, dict):
            config = self.config_class(**config)
        self.model_config = config
        # a family whose keys do not map one to one (GLM: rope_ratio, multi_query_attention) translates them itself
        d = config.to_transformer_dict() if hasattr(config, "to_transformer_dict") else config.to_dict()
        d.update(kwargs)
        if dtype is not None:
            d["params_dtype"] = d["compute_dtype"] = dtype
        d.setdefault("params_dtype", d.get("torch_dtype") or d.get("dtype") or "bfloat16")
        d.setdefault("compute_dtype", d["params_dtype"])
        if d.get("intermediate_size") is None and d.get("ffn_hidden_size") is None and d.get("multiple_of"):
            # legacy Llama configurations size the feed-forward from multiple_of / ffn_dim_multiplier
            from .llama_legacy import legacy_ffn_hidden_size
            d["intermediate_size"] = legacy_ffn_hidden_size(d["hidden_size"], None, d["multiple_of"],
                                                            d.get("ffn_dim_multiplier"))
        if d.get("seq_length") is None and d.get("max_position_embeddings"):
            d["seq_length"] = min(int(d["max_position_embeddings"]), 8192)
        tcfg = convert_to_transformer_config(d, is_mla_model=type(config).is_mla or "kv_lora_rank" in d, strict=False)
        tcfg.device = device or ("cuda" if torch.cuda.is_available() else "cpu")
        self.config = tcfg
        self.model = GPTModel(tcfg)
        self.generation_config = GenerationConfig.from_model_config(config)

    # ---- forward ----------------------------------------------------------------------------------------
    def forward(self, input_ids, labels=None, loss_mask=None, position_ids=None, attn_meta=None, **kw):
        return self.model(input_ids, labels, loss_mask, position_ids, attn_meta,
                          input_embeds=kw.get("input_embeds"))

    # make checkpoints carry the network's own names (no "model." prefix)
    def named_parameters(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True):
        for n, p in super().named_parameters(prefix, recurse, remove_duplicate):
            yield (n[len("model."):] if n.startswith("model.") else n), p

    def named_buffers(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True):
        for n, b in super().named_buffers(prefix, recurse, remove_duplicate):
            yield (n[len("model."):] if n.startswith("model.") else n), b

    # ---- name conversion hooks ----------------------------------------------------------------------------
    def convert_name(self, weight_name: str) -> str:
        return name_maps.convert_name(weight_name, self.weight_family)

    def convert_weight_dict(self, source_dict: dict, **kwargs) -> dict:
        return name_maps.hf_to_framework(source_dict, self.config, self.weight_family)

    def obtain_name_map(self, hf_keys) -> dict:
        return {k: self.convert_name(k) for k in hf_keys}

    # ---- load / save ------------------------------------------------------------------------------------------
    def load_weights(self, path: str, strict: bool = True):
        return ckpt_io.load_checkpoint(self, path, strict=strict, family=self.weight_family)

    load_checkpoint = load_weights

    @classmethod
    def from_pretrained(cls, pretrained_model_name_or_dir: str, *, config: Optional[PretrainedConfig] = None,
                        load_weights: bool = True, strict: bool = False, **kwargs) -> "PreTrainedModel":
        path = pretrained_model_name_or_dir
        if not os.path.exists(path):
            raise FileNotFoundError(f"{path} does not exist (hub download is not available offline)")
        if config is None:
            config = cls.config_class.from_pretrained(path)
        model = cls(config, **kwargs)
        if load_weights:
            try:
                ckpt_io.resolve_checkpoint(path)
                model.load_weights(path, strict=strict)
            except FileNotFoundError:
                logger.warning("no weights found under %s: the model keeps its random initialisation", path)
        model.apply_quantization_config()
        return model

    def apply_quantization_config(self, quantization_config: Optional[dict] = None, act_stats=None) -> int:
        """Quantise the (loaded) model as its configuration's ``quantization_config`` says (``quant_method``: ``rtn``,
        ``ptq``, ``smooth_quant`` or ``fp8``); returns the number of converted layers. Training modes leave the model
        as it is: the quantised layers are inference-only."""
        qc = quantization_config or getattr(self.model_config, "quantization_config", None)
        if not qc or os.environ.get("RUN_MODE", "predict") in ("train", "finetune"):
            return 0
        from ..modules.quantizers import AutoQuantizer
        n = AutoQuantizer.from_config(dict(qc)).quantize(self, act_stats)
        logger.info("quantization_config %s: %d layers converted", dict(qc).get("quant_method"), n)
        return n

    def save_pretrained(self, save_directory: str, max_shard_size: str = "5GB", hf_names: bool = False, **kw):
        size = _parse_size(max_shard_size)
        ckpt_io.save_pretrained_dir(self, save_directory, self.model_config.to_dict(), size, hf_names, self.weight_family)

    def check_pipeline_stage(self, pipeline_stage: Optional[int] = None, pp_interleave_num: Optional[int] = None):
        """A pipeline layout needs at least one layer per stage, and per virtual stage when interleaved (reference
        ``models/modeling_utils.py:317-341``). Sizes default to the model's configuration."""
        cfg = self.config
        pp = int(pipeline_stage or getattr(cfg, "pipeline_model_parallel_size", 1) or 1)
        vpp = int(pp_interleave_num or getattr(cfg, "virtual_pipeline_model_parallel_size", None) or 1)
        if pp <= 1:
            return
        layers = getattr(cfg, "num_layers", None)
        if layers is None:
            raise ValueError("num_layers is not set: the pipeline_stage check needs it")
        if layers < pp:
            raise ValueError(f"num_layers must be at least pipeline_stage, got num_layers ({layers}) < pp ({pp})")
        if vpp > 1 and pp * vpp > layers:
            raise ValueError(f"num_layers must be at least pp * pp_interleave_num, got num_layers {layers} and "
                             f"pp * pp_interleave_num = {pp * vpp}")

    def num_parameters(self) -> int:
        return sum(p.numel() for p in self.parameters())


def _parse_size(s) -> int:
    if isinstance(s, int):
        return s
    s = str(s).upper()
    for unit, mul in (("GB", 1 << 30), ("MB", 1 << 20), ("KB", 1 << 10)):
        if s.endswith(unit):
            return int(float(s[:-2]) * mul)
    return int(s)


shard_checkpoint = ckpt_io.shard_checkpoint
