"""Generation hyper-parameters (defaults of the reference's ``generation/generation_config.py:146-186``)."""
from __future__ import annotations

import copy
import json
from typing import List, Optional, Union


class GenerationConfig:
    """Generation settings (reference ``generation/generation_config.py``): ``max_length`` / ``max_new_tokens``,
    ``do_sample``, ``top_k``, ``top_p``, ``temperature``, repetition / frequency / presence penalties, ``num_beams``,
    ``eos_token_id`` (int or list), ``pad_token_id``, ``chunk_prefill_size``, ``parallel_decoding``,
    ``use_cuda_graph``. ``update(**kw)`` overrides fields, ``to_dict()`` / ``from_model_config()`` convert."""

    def __init__(self, **kwargs):
        self.max_length = kwargs.pop("max_length", kwargs.pop("max_decode_length", 20))
        self.max_new_tokens = kwargs.pop("max_new_tokens", None)
        self.min_length = kwargs.pop("min_length", 0)
        self.min_new_tokens = kwargs.pop("min_new_tokens", None)
        self.do_sample = kwargs.pop("do_sample", False)
        self.use_past = kwargs.pop("use_past", True)
        self.num_beams = kwargs.pop("num_beams", 1)
        self.temperature = kwargs.pop("temperature", 1.0)
        self.top_k = kwargs.pop("top_k", 50)
        self.top_p = kwargs.pop("top_p", 1.0)
        self.repetition_penalty = kwargs.pop("repetition_penalty", 1.0)
        self.frequency_penalty = kwargs.pop("frequency_penalty", 0.0)
        self.presence_penalty = kwargs.pop("presence_penalty", 0.0)
        self.encoder_repetition_penalty = kwargs.pop("encoder_repetition_penalty", 1.0)
        self.renormalize_logits = kwargs.pop("renormalize_logits", False)
        self.length_penalty = kwargs.pop("length_penalty", 1.0)
        self.early_stopping = kwargs.pop("early_stopping", False)
        self.num_return_sequences = kwargs.pop("num_return_sequences", 1)
        self.output_scores = kwargs.pop("output_scores", False)
        self.output_logits = kwargs.pop("output_logits", False)
        self.return_dict_in_generate = kwargs.pop("return_dict_in_generate", False)
        self.pad_token_id = kwargs.pop("pad_token_id", None)
        self.bos_token_id = kwargs.pop("bos_token_id", None)
        self.eos_token_id: Optional[Union[int, List[int]]] = kwargs.pop("eos_token_id", None)
        self.parallel_decoding = kwargs.pop("parallel_decoding", None)
        self.chunk_prefill_size = kwargs.pop("chunk_prefill_size", None)
        # capture the decode step in a CUDA graph (single-GPU models; falls back to eager launches otherwise)
        self.use_cuda_graph = kwargs.pop("use_cuda_graph", False)
        # with use_cuda_graph: pick the tokens and advance the decode state on the device and read the tokens back once
        # per ``device_loop_steps`` steps (greedy and plain temperature sampling; other settings keep the host loop)
        self.device_loop = kwargs.pop("device_loop", True)
        self.device_loop_steps = kwargs.pop("device_loop_steps", 16)
        self.seed = kwargs.pop("seed", None)
        self._extra = dict(kwargs)

    @classmethod
    def from_model_config(cls, model_config) -> "GenerationConfig":
        d = model_config.to_dict() if hasattr(model_config, "to_dict") else dict(model_config)
        keys = cls().to_dict().keys()
        return cls(**{k: v for k, v in d.items() if k in keys or k == "max_decode_length"})

    def update(self, **kwargs):
        unused = {}
        for k, v in kwargs.items():
            if hasattr(self, k):
                setattr(self, k, v)
            else:
                unused[k] = v
        return unused

    def to_dict(self) -> dict:
        return {k: copy.deepcopy(v) for k, v in vars(self).items() if not k.startswith("_")}

    def to_json_string(self) -> str:
        return json.dumps(self.to_dict(), indent=2, sort_keys=True)

    def eos_ids(self) -> List[int]:
        if self.eos_token_id is None:
            return []
        return list(self.eos_token_id) if isinstance(self.eos_token_id, (list, tuple)) else [int(self.eos_token_id)]

    def __repr__(self):
        return f"GenerationConfig {self.to_json_string()}"
