"""Cross-field validation of a full configuration before a run starts.

Rules follow the reference's ``tools/check_rules.py`` (:82-363): batch size vs data parallel, device count vs
dp·tp·cp·pp, pipeline only for training, context-parallel algorithm vs head counts, MoE expert parallel vs data
parallel, sequence parallel needs tensor parallel, recompute/swap exclusivity.
"""
from __future__ import annotations

from .logger import logger
from .utils import get_real_group_size


def _model_cfg(config):
    model = config.get("model") or {}
    return model.get("model_config") or {}


def check_parallel_config(config):
    par = config.get("parallel_config") or {}
    dp, tp = int(par.get("data_parallel", 1) or 1), int(par.get("model_parallel", 1) or 1)
    cp, pp = int(par.get("context_parallel", 1) or 1), int(par.get("pipeline_stage", 1) or 1)
    ep = int(par.get("expert_parallel", 1) or 1)
    if config.get("use_parallel"):
        world = get_real_group_size()
        if dp * tp * cp * pp != world:
            raise ValueError(f"data_parallel({dp}) * model_parallel({tp}) * context_parallel({cp}) * "
                             f"pipeline_stage({pp}) must equal the number of devices ({world})")
    if par.get("use_seq_parallel") and tp <= 1:
        logger.warning("use_seq_parallel has no effect without model_parallel > 1; it is switched off")
        par["use_seq_parallel"] = False
    if par.get("use_seq_parallel") and cp > 1:
        logger.warning("sequence parallel is ignored when context_parallel > 1")
    run_mode = config.get("run_mode")
    if pp > 1 and run_mode not in ("train", "finetune"):
        raise ValueError("pipeline_stage > 1 is only supported for training")
    mb = int(par.get("micro_batch_num", 1) or 1)
    if pp > 1 and mb < pp:
        raise ValueError(f"micro_batch_num ({mb}) must be at least pipeline_stage ({pp})")
    if ep > 1 and (dp * tp * cp) % ep != 0:
        raise ValueError(f"expert_parallel ({ep}) must divide data_parallel*model_parallel*context_parallel ({dp * tp * cp})")
    mc = _model_cfg(config)
    heads = mc.get("num_heads") or mc.get("num_attention_heads")
    if heads:
        if heads % tp:
            raise ValueError(f"num_heads ({heads}) must be divisible by model_parallel ({tp})")
        algo = par.get("context_parallel_algo", "colossalai_cp")
        if cp > 1 and algo == "ulysses_cp" and heads % (cp * tp):
            raise ValueError("ulysses_cp needs num_heads divisible by context_parallel * model_parallel")
        if cp > 1 and algo == "hybrid_cp":
            ds = int(par.get("ulysses_degree_in_cp", 1) or 1)
            if cp % ds or heads % (ds * tp):
                raise ValueError("hybrid_cp needs ulysses_degree_in_cp to divide context_parallel and the head count")
    seq = mc.get("seq_length")
    if seq and cp > 1 and seq % (cp * 2):
        raise ValueError(f"seq_length ({seq}) must be divisible by 2*context_parallel ({2 * cp})")


def check_runner_config(config):
    runner = config.get("runner_config") or {}
    bs = int(runner.get("batch_size", 1) or 1)
    if bs < 1:
        raise ValueError("runner_config.batch_size must be positive")
    ga = int(runner.get("gradient_accumulation_steps", 1) or 1)
    pp = int((config.get("parallel_config") or {}).get("pipeline_stage", 1) or 1)
    if ga > 1 and pp > 1:
        logger.warning("gradient_accumulation_steps is ignored with pipeline parallelism; use micro_batch_num")
    return bs


def check_recompute_and_swap(config):
    rec, swap = config.get("recompute_config") or {}, config.get("swap_config") or {}
    if swap.get("swap") and rec.get("recompute") is True:
        raise ValueError("full recompute and activation swap cannot both be enabled")


def check_model_config(config):
    mc = _model_cfg(config)
    if config.get("run_mode") in ("predict", "eval") and mc.get("use_flash_attention") is False:
        logger.info("flash attention is always used on CUDA; use_flash_attention=False is ignored")
    if mc.get("use_ring_attention") and (mc.get("use_attn_mask_compression") or mc.get("use_eod_attn_mask_compression")):
        raise ValueError("use_ring_attention cannot be combined with attention-mask compression")


def check_rules(config, mode: str = "train", **kwargs):
    """Raise on inconsistent settings; may normalise a few keys in place."""
    check_parallel_config(config)
    check_runner_config(config)
    check_recompute_and_swap(config)
    check_model_config(config)
    return config
