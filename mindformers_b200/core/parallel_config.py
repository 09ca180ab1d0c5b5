"""YAML ``parallel_config`` / ``recompute_config`` / ``swap_config`` / ``moe_config`` sections as objects.

Reference: ``mindformers/core/parallel_config.py:28-76`` (``build_parallel_config``: dict sections →
``TransformerOpParallelConfig`` / ``TransformerRecomputeConfig`` / ``TransformerSwapConfig`` / ``MoEConfig``; a
pipeline of more than one stage forces ``vocab_emb_dp=False``) and ``modules/transformer/op_parallel_config.py``.
The objects carry the reference's field names; ``to_parallel_state_kwargs`` maps them onto
``parallel_state.initialize_model_parallel``.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field, is_dataclass
from enum import Enum
from typing import Any, Dict, List, Optional, Union


class ContextParallelAlgo(Enum):
    """How the sequence is split over the context-parallel ranks (``op_parallel_config.py:250``): K/V exchange
    between sequence shards, head all-to-all, or the first inside groups of the second."""
    COLOSSALAI_CP = "colossalai_cp"
    ULYSSES_CP = "ulysses_cp"
    HYBRID_CP = "hybrid_cp"


@dataclass
class OpParallelConfig:
    """Degrees that a single operator is split by (``op_parallel_config.py:48``): data, model (tensor), context."""
    data_parallel: int = 1
    model_parallel: int = 1
    context_parallel: int = 1
    use_seq_parallel: bool = False
    select_recompute: bool = False
    context_parallel_algo: str = "colossalai_cp"

    def __post_init__(self):
        for name in ("data_parallel", "model_parallel", "context_parallel"):
            v = getattr(self, name)
            if not isinstance(v, int) or v < 1:
                raise ValueError(f"{name} must be a positive integer, got {v!r}")
        ContextParallelAlgo(self.context_parallel_algo)          # raises on an unknown name

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)


@dataclass
class _PipeLineConfig:
    """Pipeline degrees (``op_parallel_config.py:132``)."""
    pipeline_stage: int = 1
    micro_batch_num: int = 1
    seq_split_num: int = 1

    def __post_init__(self):
        for name in ("pipeline_stage", "micro_batch_num", "seq_split_num"):
            v = getattr(self, name)
            if not isinstance(v, int) or v < 1:
                raise ValueError(f"{name} must be a positive integer, got {v!r}")


@dataclass
class TransformerRecomputeConfig:
    """``recompute_config`` section: full (``recompute``), selective (``select_recompute`` patterns) and
    communication recomputation switches."""

    recompute: Union[bool, list] = False
    select_recompute: Union[bool, list] = False
    parallel_optimizer_comm_recompute: bool = False
    select_comm_recompute: Union[bool, list] = False
    mp_comm_recompute: bool = True
    recompute_slice_activation: bool = False
    select_recompute_exclude: Union[bool, list] = False
    select_comm_recompute_exclude: Union[bool, list] = False


@dataclass
class TransformerSwapConfig:
    """``swap_config`` section: which layers / operators keep their activations in host memory and how far ahead they
    are fetched back."""

    swap: bool = False
    default_prefetch: int = 1
    layer_swap: Optional[list] = None
    op_swap: Optional[list] = None


@dataclass
class MoEParallelConfig:
    """Degrees seen by an MoE layer: data, model, expert, context."""

    data_parallel: int = 1
    model_parallel: int = 1
    expert_parallel: int = 1
    context_parallel: int = 1


@dataclass
class TransformerOpParallelConfig:
    """``parallel_config`` section as an object (reference ``modules/transformer/transformer.py:535-700``): data /
    model / context / expert / pipeline degrees, micro-batches, sequence parallelism, context-parallel algorithm,
    with the recompute and swap configurations attached."""

    data_parallel: int = 1
    model_parallel: int = 1
    context_parallel: int = 1
    expert_parallel: int = 1
    pipeline_stage: int = 1
    micro_batch_num: int = 1
    seq_split_num: int = 1
    use_seq_parallel: bool = False
    optimizer_shard: Optional[bool] = None
    gradient_aggregation_group: int = 4
    vocab_emb_dp: bool = True
    context_parallel_algo: str = "colossalai_cp"
    ulysses_degree_in_cp: int = 1
    mem_coeff: float = 0.1
    virtual_pipeline_stage: Optional[int] = None
    recompute: TransformerRecomputeConfig = field(default_factory=TransformerRecomputeConfig)
    swap: TransformerSwapConfig = field(default_factory=TransformerSwapConfig)

    def __post_init__(self):
        for name in ("data_parallel", "model_parallel", "context_parallel", "expert_parallel", "pipeline_stage",
                     "micro_batch_num", "seq_split_num", "ulysses_degree_in_cp"):
            v = getattr(self, name)
            if not isinstance(v, int) or v < 1:
                raise ValueError(f"parallel_config.{name} must be a positive integer, got {v!r}")
        if self.context_parallel_algo not in ("colossalai_cp", "ulysses_cp", "hybrid_cp"):
            raise ValueError(f"context_parallel_algo {self.context_parallel_algo!r} is not one of "
                             "colossalai_cp / ulysses_cp / hybrid_cp")
        if self.pipeline_stage > 1:
            self.vocab_emb_dp = False           # the embedding is model-parallel once the model is staged

    @property
    def dp_mp_config(self) -> OpParallelConfig:
        return OpParallelConfig(self.data_parallel, self.model_parallel, self.context_parallel, self.use_seq_parallel,
                                bool(self.recompute.select_recompute), self.context_parallel_algo)

    @property
    def pipeline_config(self) -> _PipeLineConfig:
        return _PipeLineConfig(self.pipeline_stage, self.micro_batch_num, self.seq_split_num)

    @property
    def moe_parallel_config(self) -> MoEParallelConfig:
        return MoEParallelConfig(self.data_parallel, self.model_parallel, self.expert_parallel, self.context_parallel)

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)

    def to_parallel_state_kwargs(self) -> Dict[str, Any]:
        """Arguments of ``parallel_state.initialize_model_parallel`` for these degrees."""
        kw = dict(tensor_model_parallel_size=self.model_parallel, pipeline_model_parallel_size=self.pipeline_stage,
                  context_parallel_size=self.context_parallel, expert_model_parallel_size=self.expert_parallel)
        if self.virtual_pipeline_stage and self.virtual_pipeline_stage > 1:
            kw["virtual_pipeline_model_parallel_size"] = self.virtual_pipeline_stage
        return kw

    def cp_comm_type(self) -> str:
        return {"colossalai_cp": "p2p", "ulysses_cp": "a2a", "hybrid_cp": "a2a+p2p"}[self.context_parallel_algo]


@dataclass
class EmbeddingOpParallelConfig:
    """Degrees of the vocabulary embedding (reference ``modules/transformer/transformer.py:87``): with ``vocab_emb_dp``
    the table is replicated and the lookup is data-parallel, otherwise its rows are split ``model_parallel`` ways."""
    data_parallel: int = 1
    model_parallel: int = 1
    context_parallel: int = 1
    use_seq_parallel: bool = False
    select_recompute: bool = False
    vocab_emb_dp: bool = True

    def __post_init__(self):
        if not isinstance(self.vocab_emb_dp, bool):
            raise TypeError(f"vocab_emb_dp must be a bool, got {type(self.vocab_emb_dp).__name__}")
        self.dp_mp_config                                   # validates the degrees

    @property
    def dp_mp_config(self) -> OpParallelConfig:
        return OpParallelConfig(self.data_parallel, self.model_parallel, self.context_parallel, self.use_seq_parallel,
                                self.select_recompute)

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)


default_transformer_config = TransformerOpParallelConfig()
default_recompute_config = TransformerRecomputeConfig()
default_moe_parallel_config = MoEParallelConfig()
default_dpmp_config = OpParallelConfig()


def build_parallel_config(config) -> TransformerOpParallelConfig:
    """Replace the dict sections of ``config`` (a ``MindFormerConfig`` or dict) by objects and return the parallel one.
    Sets ``config.parallel_config``, ``config.recompute_config``, ``config.swap_config`` in place."""
    get = (lambda k: config.get(k)) if hasattr(config, "get") else (lambda k: getattr(config, k, None))
    rc = get("recompute_config")
    recompute = rc if isinstance(rc, TransformerRecomputeConfig) else TransformerRecomputeConfig(
        **{k: v for k, v in dict(rc or {}).items() if k in TransformerRecomputeConfig.__dataclass_fields__})
    sc = get("swap_config")
    swap = sc if isinstance(sc, TransformerSwapConfig) else TransformerSwapConfig(
        **{k: v for k, v in dict(sc or {}).items() if k in TransformerSwapConfig.__dataclass_fields__})
    pc = get("parallel_config")
    if isinstance(pc, TransformerOpParallelConfig):
        par = pc
        par.recompute, par.swap = recompute, swap
    else:
        fields = TransformerOpParallelConfig.__dataclass_fields__
        par = TransformerOpParallelConfig(recompute=recompute, swap=swap,
                                          **{k: v for k, v in dict(pc or {}).items()
                                             if k in fields and k not in ("recompute", "swap") and v is not None})
    for key, val in (("parallel_config", par), ("recompute_config", recompute), ("swap_config", swap)):
        if isinstance(config, dict):
            config[key] = val
        else:
            setattr(config, key, val)
    return par


def _as_dict(obj) -> Dict[str, Any]:
    return obj.to_dict() if hasattr(obj, "to_dict") else asdict(obj)


def _diff_dict(obj) -> Dict[str, Any]:
    """The fields of a configuration object that differ from its class defaults."""
    if hasattr(obj, "to_diff_dict"):
        return obj.to_diff_dict()
    full, base = _as_dict(obj), _as_dict(type(obj)())
    return {k: v for k, v in full.items() if base.get(k) != v}


def reset_parallel_config(config, reset_diff_config: bool = True):
    """Inverse of ``build_parallel_config``: turn the ``moe_config`` / ``recompute_config`` / ``parallel_config`` objects
    of ``config`` back into plain dicts (only the non-default fields with ``reset_diff_config``), so that the
    configuration can be written to YAML or rebuilt (reference ``core/parallel_config.py:79``)."""
    get = (lambda k: config.get(k)) if hasattr(config, "get") else (lambda k: getattr(config, k, None))

    def put(k, v):
        if hasattr(config, "__setitem__"):
            config[k] = v
        else:
            setattr(config, k, v)

    for key in ("moe_config", "recompute_config", "swap_config", "parallel_config"):
        obj = get(key)
        if obj is None or isinstance(obj, dict) or not (hasattr(obj, "to_dict") or is_dataclass(obj)):
            continue
        d = _diff_dict(obj) if reset_diff_config else _as_dict(obj)
        if key == "parallel_config":
            d.pop("recompute", None)
            d.pop("swap", None)
        put(key, d)
    return config
