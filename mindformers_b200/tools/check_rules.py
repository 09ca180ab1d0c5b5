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


def check_mode(config, mode: str, network=None, dataset=None, task=None):
    """Rules that depend on the run mode (reference ``_check_mode`` :48-116): generation tasks need a batch that splits
    over the data-parallel ranks; pipeline stages are a training-only layout."""
    par = config.get("parallel_config") or {}
    dp, pp = int(par.get("data_parallel", 1) or 1), int(par.get("pipeline_stage", 1) or 1)
    if mode in ("predict", "eval") and pp > 1:
        raise ValueError(f"pipeline_stage > 1 is a training layout: set pipeline_stage to 1 for {mode}")
    if task == "text_generation" or mode == "predict":
        bs = None
        if dataset is not None and hasattr(dataset, "get_batch_size"):
            bs = dataset.get_batch_size()
        elif network is not None and getattr(getattr(network, "config", None), "batch_size", None):
            bs = network.config.batch_size
        else:
            bs = _model_cfg(config).get("batch_size") or (config.get("runner_config") or {}).get("batch_size")
        bs = 1 if bs is None else int(bs)
        if config.get("use_parallel") and bs % dp:
            raise ValueError(f"batch_size must be divisible by data_parallel: {bs} % {dp} = {bs % dp}")


def check_keyword_gen_dataset(config, mode: str, network=None, dataset=None):
    """ADGen-style keyword-generation data (reference :212-272): in training ``seq_length`` must equal
    ``max_source_length + max_target_length + 1``; evaluation with the generation metric needs ``seq_length ==
    max_source_length``, with the perplexity metric the training relation and the training phase of the loader."""
    if network is not None or dataset is not None:
        return                                   # objects built by the caller are taken as they are
    seq = _model_cfg(config).get("seq_length")
    if not seq:
        return
    train_ds, eval_ds = config.get("train_dataset") or {}, config.get("eval_dataset") or {}

    def is_adgen(ds):
        return ((ds.get("data_loader") or {}).get("type")) == "ADGenDataLoader"

    def need(kind, ds, where):
        src, tgt = ds.get("max_source_length"), ds.get("max_target_length")
        if src is None or tgt is None:
            return
        if kind == "train" and src + tgt + 1 != seq:
            raise ValueError(f"make sure seq_length = max_source_length + max_target_length + 1 in {where}: "
                             f"seq_length={seq}, max_source_length={src}, max_target_length={tgt}")
        if kind == "eval" and src != seq:
            raise ValueError(f"make sure seq_length = max_source_length in {where}: seq_length={seq}, max_source_length={src}")

    metrics = config.get("metric") or []
    metrics = [metrics] if isinstance(metrics, dict) else list(metrics)
    kinds = [m.get("type") for m in metrics if isinstance(m, dict)]
    if mode in ("train", "finetune") and is_adgen(train_ds):
        need("train", train_ds, "train_dataset")
        if config.get("do_eval") and is_adgen(eval_ds):
            if "ADGENMetric" in kinds:
                need("eval", eval_ds, "eval_dataset")
            if "PerplexityMetric" in kinds:
                need("train", eval_ds, "eval_dataset")
    if mode == "eval" and is_adgen(eval_ds):
        if "ADGENMetric" in kinds:
            need("eval", eval_ds, "eval_dataset")
        if "PerplexityMetric" in kinds:
            need("train", eval_ds, "eval_dataset")
    if "PerplexityMetric" in kinds and eval_ds and (eval_ds.get("data_loader") or {}).get("phase") not in (None, "train"):
        logger.warning("PerplexityMetric scores teacher-forced tokens: eval_dataset.data_loader.phase is set to 'train'")
        eval_ds["data_loader"]["phase"] = "train"
        task_cfg = ((config.get("eval_dataset_task") or {}).get("dataset_config") or {}).get("data_loader")
        if isinstance(task_cfg, dict):
            task_cfg["phase"] = "train"


def _layer_list_ok(value, key, pp):
    """A recompute / swap selector is a bool, a list of per-stage layer counts (at most one per pipeline stage, all
    integers) or, with swap, a mapping ``operator pattern -> list of layers``."""
    if isinstance(value, (list, tuple)):
        if any(isinstance(x, bool) or not isinstance(x, int) for x in value):
            if all(isinstance(x, str) for x in value):
                return                           # module / operator patterns (select_recompute: ["mlp", "core_attention"])
            raise ValueError(f"the elements of {key} must all be int (layers per stage) or all be str (patterns), got {value}")
        if len(value) > pp:
            raise ValueError(f"{key} has {len(value)} entries for {pp} pipeline stage(s): at most one per stage")
    elif isinstance(value, dict):
        for op, layers in value.items():
            if not isinstance(op, str):
                raise ValueError(f"the keys of {key} must be operator patterns (str), got {type(op).__name__}")
            if not isinstance(layers, (list, tuple, bool)):
                raise ValueError(f"the layers of {key}[{op!r}] must be a list, got {type(layers).__name__}")
    elif value is not None and not isinstance(value, bool):
        raise ValueError(f"{key} must be a bool, a list or a mapping, got {type(value).__name__}")


def check_recompute_shapes(config):
    """Shape rules of ``recompute_config`` and ``swap_config`` (reference :285-360)."""
    rec, swap = config.get("recompute_config") or {}, config.get("swap_config") or {}
    pp = int((config.get("parallel_config") or {}).get("pipeline_stage", 1) or 1)
    for key in ("recompute", "select_recompute", "select_comm_recompute"):
        _layer_list_ok(rec.get(key), key, pp)
    flag = swap.get("swap", False)
    if not isinstance(flag, bool):
        raise ValueError(f"swap_config.swap must be a bool, got {type(flag).__name__}")
    if not flag:
        return
    prefetch = swap.get("default_prefetch", 1)
    if isinstance(prefetch, bool) or not isinstance(prefetch, int) or prefetch < 1:
        raise ValueError(f"swap_config.default_prefetch must be a positive int, got {prefetch!r}")

    def swap_list(value, key):
        if value in (None, False):
            return
        if not isinstance(value, list):
            raise ValueError(f"{key} must be a list of mappings, got {type(value).__name__}")
        for item in value:
            if not isinstance(item, dict):
                raise ValueError(f"every element of {key} must be a mapping, got {type(item).__name__}")
            _layer_list_ok(item.get("layers"), key + ".layers", pp)
            bp = item.get("backward_prefetch", prefetch)
            if isinstance(bp, bool) or not isinstance(bp, int) or bp < 1:
                raise ValueError(f"{key}.backward_prefetch must be a positive int, got {bp!r}")
    swap_list(swap.get("layer_swap"), "layer_swap")
    ops = swap.get("op_swap")
    if ops not in (None, False) and not isinstance(ops, dict):
        raise ValueError(f"swap_config.op_swap must be a mapping, got {type(ops).__name__}")
    for op, info in (ops or {}).items():
        swap_list(info, f"op_swap({op})")


def check_compatibility(config):
    """Features that need one another (reference ``_check_config_campacity`` :320-327, ``_check_moe_parallel_valid``)."""
    mc, par = _model_cfg(config), config.get("parallel_config") or {}
    fgi = int(mc.get("fine_grain_interleave") or 1)
    cp = int(par.get("context_parallel", 1) or 1)
    if fgi > 1 and not par.get("use_seq_parallel") and cp <= 1:
        raise ValueError("fine_grain_interleave > 1 without context parallelism needs use_seq_parallel: True")
    experts = mc.get("num_experts") or mc.get("n_routed_experts") or (config.get("moe_config") or {}).get("expert_num")
    ep = int(par.get("expert_parallel", 1) or 1)
    if experts and ep > 1 and int(experts) % ep:
        raise ValueError(f"the number of experts ({experts}) must be divisible by expert_parallel ({ep})")
    seq_split = int(par.get("seq_split_num", 1) or 1)
    if seq_split > 1 and int(par.get("pipeline_stage", 1) or 1) <= 1:
        raise ValueError("seq_split_num > 1 (sequence pipeline) needs pipeline_stage > 1")


YAML_MAX_NESTING_DEPTH = 10


def get_yaml_ast_depth(node, depth: int = 0) -> int:
    """Nesting depth of a parsed YAML node tree (``yaml.compose``)."""
    import yaml
    if isinstance(node, yaml.MappingNode):
        return max([get_yaml_ast_depth(v, depth + 1) for _, v in node.value] + [depth + 1])
    if isinstance(node, yaml.SequenceNode):
        return max([get_yaml_ast_depth(v, depth + 1) for v in node.value] + [depth + 1])
    return depth


def check_yaml_depth_before_loading(yaml_str: str, max_depth: int = YAML_MAX_NESTING_DEPTH):
    """Refuse a YAML text nested deeper than ``max_depth`` before it is turned into objects (reference :374-391: a guard
    against crafted inputs that exhaust the loader)."""
    import yaml
    node = yaml.compose(yaml_str, Loader=yaml.SafeLoader)
    if node is not None and get_yaml_ast_depth(node) > max_depth:
        raise ValueError(f"the YAML text is nested deeper than {max_depth} levels")


def check_rules(config, mode: str = "train", **kwargs):
    """Raise on inconsistent settings; may normalise a few keys in place. ``kwargs``: ``network``, ``dataset``, ``task``
    when the caller built those itself."""
    check_mode(config, mode, kwargs.get("network"), kwargs.get("dataset"), kwargs.get("task"))
    check_parallel_config(config)
    check_runner_config(config)
    check_keyword_gen_dataset(config, mode, kwargs.get("network"), kwargs.get("dataset"))
    check_recompute_and_swap(config)
    check_recompute_shapes(config)
    check_compatibility(config)
    check_model_config(config)
    return config
