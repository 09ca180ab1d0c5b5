import os
import textwrap

import pytest

from mindformers_b200.tools.register import (ConfigTemplate, MindFormerConfig, MindFormerModuleType,
                                             MindFormerRegister, set_use_legacy)
from mindformers_b200.tools.register.config import ActionDict, parse_value


def _write(tmp_path, name, text):
    p = tmp_path / name
    p.write_text(textwrap.dedent(text))
    return str(p)


def test_yaml_inheritance_and_attribute_access(tmp_path):
    _write(tmp_path, "base.yaml", """
        seed: 7
        runner_config: {batch_size: 2, epochs: 3}
        model: {model_config: {hidden_size: 64, num_layers: 2}}
    """)
    child = _write(tmp_path, "child.yaml", """
        base_config: base.yaml
        runner_config: {batch_size: 8}
        model: {model_config: {num_layers: 4}}
    """)
    cfg = MindFormerConfig(child)
    assert cfg.seed == 7
    assert cfg.runner_config.batch_size == 8 and cfg.runner_config.epochs == 3
    assert cfg.model.model_config.hidden_size == 64 and cfg.model.model_config.num_layers == 4
    assert cfg.not_there is None
    cfg.merge_from_dict({"model.model_config.num_layers": 6, "new.section.key": 1})
    assert cfg.get_value("model.model_config.num_layers") == 6
    assert cfg.new.section.key == 1
    cfg.set_value("runner_config.epochs", 9)
    assert cfg.to_dict()["runner_config"]["epochs"] == 9


def test_circular_base_config_is_rejected(tmp_path):
    _write(tmp_path, "a.yaml", "base_config: b.yaml\nx: 1\n")
    b = _write(tmp_path, "b.yaml", "base_config: a.yaml\ny: 2\n")
    with pytest.raises(ValueError):
        MindFormerConfig(b)


def test_parse_value_and_action_dict():
    assert parse_value("1e-3") == 1e-3 and parse_value("True") is True and parse_value("[1,2]") == [1, 2]
    assert parse_value("abc") == "abc" and parse_value("None") is None
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--options", nargs="+", action=ActionDict)
    ns = ap.parse_args(["--options", "a.b=3", "c=hello"])
    assert ns.options == {"a.b": 3, "c": "hello"}


def test_template_defaults_and_strict_sections():
    cfg = {"run_mode": "train", "parallel_config": {"data_parallel": 4}, "optimizer": {"type": "AdamW", "learning_rate": 1e-3}}
    ConfigTemplate.apply_template(cfg)
    assert cfg["parallel_config"]["model_parallel"] == 1 and cfg["parallel_config"]["data_parallel"] == 4
    assert cfg["optimizer"]["betas"] == [0.9, 0.999] and cfg["optimizer"]["learning_rate"] == 1e-3
    assert cfg["seed"] == 1 and cfg["callbacks"][0]["type"] == "MFLossMonitor"
    with pytest.raises(KeyError):
        ConfigTemplate.apply_template({"run_mode": "train", "parallel_config": {"bogus": 1}})
    # predict mode drops the training sections; mcore mode drops moe_config
    cfg = {"run_mode": "predict", "use_legacy": False, "optimizer": {"type": "AdamW"}, "moe_config": {"expert_num": 4}}
    ConfigTemplate.apply_template(cfg)
    assert "optimizer" not in cfg and "moe_config" not in cfg and "processor" in cfg


def test_registry_roundtrip_and_mcore_prefix():
    @MindFormerRegister.register(MindFormerModuleType.TOOLS, alias="_probe_tool")
    class Probe:
        def __init__(self, a=1, b=2):
            self.a, self.b = a, b

    assert MindFormerRegister.is_exist(MindFormerModuleType.TOOLS, "_probe_tool")
    inst = MindFormerRegister.get_instance_from_cfg({"type": "_probe_tool", "a": 5}, MindFormerModuleType.TOOLS,
                                                    default_args={"b": 9})
    assert (inst.a, inst.b) == (5, 9)
    with pytest.raises(ValueError):
        MindFormerRegister.get_cls(MindFormerModuleType.TOOLS, "_missing_")

    @MindFormerRegister.register(MindFormerModuleType.MODELS, alias="_ProbeModel", legacy=False)
    class ProbeModel:
        pass

    set_use_legacy(False)
    try:
        assert MindFormerRegister.get_cls(MindFormerModuleType.MODELS, "_ProbeModel") is ProbeModel
        assert "mcore__ProbeModel" in MindFormerRegister.registry[MindFormerModuleType.MODELS]
    finally:
        set_use_legacy(True)


def test_auto_register_from_register_path(tmp_path, monkeypatch):
    pkg = tmp_path / "plug"
    pkg.mkdir()
    (pkg / "mod.py").write_text("class Extra:\n    value = 3\n")
    monkeypatch.setenv("REGISTER_PATH", str(tmp_path))
    cls = MindFormerRegister.auto_register("plug.mod.Extra", MindFormerModuleType.TOOLS)
    assert cls.value == 3 and MindFormerRegister.get_cls(MindFormerModuleType.TOOLS, "Extra") is cls


def test_parallel_config_objects_and_cpu_masks():
    from mindformers_b200.core.parallel_config import build_parallel_config
    from mindformers_b200.utils.bit_array import BitArray
    from mindformers_b200.utils.cpu_affinity import cores_for_rank, format_cpu_list, parse_cpu_list
    import pytest as _pytest
    cfg = {"parallel_config": {"data_parallel": 2, "model_parallel": 4, "pipeline_stage": 2, "micro_batch_num": 8,
                               "use_seq_parallel": True, "context_parallel_algo": "ulysses_cp"},
           "recompute_config": {"recompute": [2, 1], "select_recompute": False}}
    par = build_parallel_config(cfg)
    assert par.model_parallel == 4 and par.vocab_emb_dp is False            # staged model: model-parallel embedding
    assert par.recompute.recompute == [2, 1] and cfg["recompute_config"] is par.recompute
    assert par.to_parallel_state_kwargs()["pipeline_model_parallel_size"] == 2 and par.cp_comm_type() == "a2a"
    with _pytest.raises(ValueError):
        build_parallel_config({"parallel_config": {"model_parallel": 0}})
    bits = BitArray(64).load_from_str("0000000f,000000f0")
    assert bits.get_marked_index() == [4, 5, 6, 7, 32, 33, 34, 35] and bits.to_mask_str() == "0000000f,000000f0"
    assert (bits - BitArray.from_indices([4, 32])).count() == 6
    assert parse_cpu_list("0-3,8,10-11") == [0, 1, 2, 3, 8, 10, 11] and format_cpu_list([0, 1, 2, 3, 8, 10, 11]) == "0-3,8,10-11"
    numa = {0: list(range(0, 16)), 1: list(range(16, 32))}
    assert cores_for_rank(1, 4, range(32), reserved=[0], numa=numa, gpu_node=0) == list(range(8, 15))
    assert cores_for_rank(3, 4, range(32)) == list(range(24, 32))
    assert cores_for_rank(2, 4, range(32), numa=numa, gpu_node=1) == list(range(16, 24))


def test_misc_utils(tmp_path):
    import warnings
    from mindformers_b200.tools.generic import add_model_info_to_auto_map, is_experimental_mode
    from mindformers_b200.utils.decorators import deprecated
    from mindformers_b200.utils.import_utils import is_package_available, requires_backends
    import pytest as _pytest

    @deprecated("use g", version="1.2")
    def f(x):
        return x + 1

    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        assert f(1) == 2
    assert "deprecated since 1.2: use g" in str(w[0].message)
    assert is_package_available("torch") and not is_package_available("surely_not_installed_pkg")
    with _pytest.raises(ImportError):
        requires_backends(f, ["surely_not_installed_pkg"])
    (tmp_path / "hf").mkdir()
    (tmp_path / "hf" / "config.json").write_text("{}")
    (tmp_path / "origin").mkdir()
    (tmp_path / "origin" / "model.yaml").write_text("a: 1")
    assert is_experimental_mode(str(tmp_path / "hf")) and not is_experimental_mode(str(tmp_path / "origin"))
    assert is_experimental_mode("org/model") and not is_experimental_mode("llama2_7b")
    assert add_model_info_to_auto_map({"AutoModel": "m.C"}, "org/r") == {"AutoModel": "org/r--m.C"}


def test_top_level_api_surface():
    """The names the reference documents at the package root (docs/api/api_python) resolve."""
    import mindformers_b200 as mf
    for name in ("AutoConfig", "AutoModel", "AutoModelForCausalLM", "AutoProcessor", "AutoTokenizer", "ModelRunner",
                 "Trainer", "TrainingArguments", "pipeline", "run_check", "MindFormerConfig", "MindFormerRegister",
                 "MindFormerModuleType", "GenerationConfig", "GenerationMixin", "LlamaConfig", "LlamaForCausalLM",
                 "LlamaTokenizer", "LlamaTokenizerFast", "ChatGLM3Tokenizer", "ChatGLM4Tokenizer", "PreTrainedModel",
                 "PretrainedConfig", "CausalLanguageModelDataset", "KeyWordGenDataset", "MultiTurnDataset", "LoraConfig",
                 "LoraModel", "PetConfig", "MultiModalToTextPipeline", "MFTrainOneStepCell", "MFPipelineWithLossScaleCell"):
        assert getattr(mf, name) is not None, name
    from mindformers_b200.core import AdamW, CosineWithWarmUpLR, CrossEntropyLoss, MFLossMonitor, PerplexityMetric  # noqa: F401
    from mindformers_b200.wrapper import MFTrainOneStepCell
    assert MFTrainOneStepCell.__name__ == "TrainOneStep"


def test_context_reads_parallel_speed_up_json(tmp_path):
    """Graph-compiler knobs of the reference's backend: the overlap ones select the fused kernels, the rest is listed."""
    import json
    from mindformers_b200.core.context import Context
    path = tmp_path / "parallel_speed_up.json"
    json.dump({"matmul_grad_comm_overlap": True, "dataset_broadcast_opt_level": 3, "enable_grad_comm_opt": False,
               "some_future_knob": 1}, open(path, "w"))
    cfg = {"context": {"device_target": "CPU", "ascend_config": {"parallel_speed_up_json_path": str(path)}},
           "model": {"model_config": {"hidden_size": 8}}}
    ctx = Context(cfg)
    assert ctx.parallel_speed_up["applied"] == {"matmul_grad_comm_overlap": "fused_tp_comm"}
    assert set(ctx.parallel_speed_up["ignored"]) == {"dataset_broadcast_opt_level", "enable_grad_comm_opt", "some_future_knob"}
    assert cfg["model"]["model_config"]["fused_tp_comm"] is True
    assert Context({"context": {"device_target": "CPU"}}).parallel_speed_up["path"] is None


def test_op_parallel_config_objects():
    import pytest
    from mindformers_b200.core.parallel_config import (ContextParallelAlgo, OpParallelConfig, TransformerOpParallelConfig,
                                                       _PipeLineConfig, default_dpmp_config)
    par = TransformerOpParallelConfig(data_parallel=2, model_parallel=4, context_parallel=2, pipeline_stage=2,
                                      micro_batch_num=8, context_parallel_algo="ulysses_cp", use_seq_parallel=True)
    dpmp = par.dp_mp_config
    assert (dpmp.data_parallel, dpmp.model_parallel, dpmp.context_parallel, dpmp.use_seq_parallel) == (2, 4, 2, True)
    assert ContextParallelAlgo(dpmp.context_parallel_algo) is ContextParallelAlgo.ULYSSES_CP
    assert par.pipeline_config == _PipeLineConfig(2, 8, 1) and default_dpmp_config.model_parallel == 1
    with pytest.raises(ValueError):
        OpParallelConfig(context_parallel_algo="ring_of_rings")
    with pytest.raises(ValueError):
        _PipeLineConfig(pipeline_stage=0)


def _shipped_yaml_files():
    import glob
    import os
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "configs")
    return sorted(p for p in glob.glob(os.path.join(root, "*", "*.yaml")) if "convert_config" not in p)


@pytest.mark.parametrize("path", _shipped_yaml_files(), ids=lambda p: "/".join(p.split("/")[-2:]))
def test_every_shipped_yaml_loads_validates_and_builds_a_shrunk_model(path, monkeypatch):
    """Each YAML under ``configs/`` parses, passes the cross-field rules and its ``model_config`` (shrunk to two small
    layers) builds a model of the registered family that runs a forward pass."""
    import torch
    from mindformers_b200.models import AutoModel
    from mindformers_b200.tools.check_rules import check_rules
    from mindformers_b200.tools.register import MindFormerConfig
    cfg = MindFormerConfig(path)
    assert cfg.run_mode in ("train", "finetune", "predict", "eval")
    pc = cfg.parallel_config or {}
    devices = 1
    for key in ("data_parallel", "model_parallel", "context_parallel", "pipeline_stage"):
        devices *= int(pc.get(key, 1) or 1)
    monkeypatch.setenv("WORLD_SIZE", str(devices))          # the rules compare the degrees with the launch size
    check_rules(cfg, mode=cfg.run_mode)
    mc = dict(cfg.model.model_config)
    heads = 4
    small = dict(num_hidden_layers=2, hidden_size=64, num_attention_heads=heads, intermediate_size=128, vocab_size=256,
                 max_position_embeddings=128, seq_length=64, params_dtype="float32", compute_dtype="float32")
    if mc.get("num_key_value_heads"):
        small["num_key_value_heads"] = min(int(mc["num_key_value_heads"]), heads) if int(mc["num_key_value_heads"]) < int(mc["num_attention_heads"]) else heads
    if mc.get("head_dim"):
        small["head_dim"] = 16
    for key in ("num_experts", "n_routed_experts"):
        if mc.get(key):
            small[key] = 4
            small["moe_intermediate_size"] = 32
            small["num_experts_per_tok"] = 2
    if mc.get("shared_expert_intermediate_size"):
        small["shared_expert_intermediate_size"] = 48
    if mc.get("n_group"):
        small.update(n_group=2, topk_group=1)
    if mc.get("first_k_dense_replace"):
        small["first_k_dense_replace"] = 1
    if mc.get("kv_lora_rank"):
        small.update(kv_lora_rank=32, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
                     q_lora_rank=32 if mc.get("q_lora_rank") else None)
    if mc.get("num_nextn_predict_layers"):
        small["num_nextn_predict_layers"] = 1
    for drop in ("num_blocks", "fused_tp_comm", "fused_moe_comm", "fused_cp_comm", "offset", "rope_scaling"):
        mc.pop(drop, None)
    mc.update(small)
    torch.manual_seed(0)
    model = AutoModel.from_config(mc, device="cpu").eval()
    with torch.no_grad():
        logits = model(torch.randint(0, 256, (1, 8)))
    assert logits.shape[-1] >= 256 and torch.isfinite(logits).all()


def test_cross_field_rules_of_modes_datasets_recompute_and_swap():
    from mindformers_b200.tools.check_rules import (check_compatibility, check_keyword_gen_dataset, check_mode,
                                                    check_recompute_shapes, check_yaml_depth_before_loading)
    base = {"parallel_config": {"data_parallel": 2, "pipeline_stage": 2}, "use_parallel": True,
            "model": {"model_config": {"seq_length": 64, "batch_size": 3}}}
    with pytest.raises(ValueError, match="training layout"):
        check_mode(base, "predict")
    flat = {"parallel_config": {"data_parallel": 2}, "use_parallel": True, "model": {"model_config": {"batch_size": 3}}}
    with pytest.raises(ValueError, match="divisible by data_parallel"):
        check_mode(flat, "predict")
    check_mode(flat, "train")
    # keyword-generation data: seq_length = source + target + 1 in training, = source for the generation metric
    adgen = {"model": {"model_config": {"seq_length": 193}}, "do_eval": True, "metric": [{"type": "ADGENMetric"}],
             "train_dataset": {"data_loader": {"type": "ADGenDataLoader"}, "max_source_length": 64, "max_target_length": 128},
             "eval_dataset": {"data_loader": {"type": "ADGenDataLoader"}, "max_source_length": 64, "max_target_length": 128}}
    with pytest.raises(ValueError, match="eval_dataset"):
        check_keyword_gen_dataset(adgen, "train")
    adgen["eval_dataset"]["max_source_length"] = 193
    check_keyword_gen_dataset(adgen, "train")
    adgen["train_dataset"]["max_target_length"] = 100
    with pytest.raises(ValueError, match="train_dataset"):
        check_keyword_gen_dataset(adgen, "train")
    ppl = {"model": {"model_config": {"seq_length": 8}}, "metric": {"type": "PerplexityMetric"},
           "eval_dataset": {"data_loader": {"type": "X", "phase": "eval"}}}
    check_keyword_gen_dataset(ppl, "eval")
    assert ppl["eval_dataset"]["data_loader"]["phase"] == "train"
    # recompute / swap shapes
    ok = {"parallel_config": {"pipeline_stage": 2}, "recompute_config": {"recompute": [3, 2], "select_recompute": ["mlp"]},
          "swap_config": {"swap": True, "default_prefetch": 1,
                          "layer_swap": [{"layers": [0, 1], "backward_prefetch": 2}], "op_swap": {"mlp": [{"layers": [1], "backward_prefetch": 1}]}}}
    check_recompute_shapes(ok)
    for bad, msg in (({"recompute_config": {"recompute": [1, 2, 3]}, "parallel_config": {"pipeline_stage": 2}}, "at most one per stage"),
                     ({"recompute_config": {"select_recompute": [1, "mlp"]}}, "all be int"),
                     ({"swap_config": {"swap": "yes"}}, "must be a bool"),
                     ({"swap_config": {"swap": True, "default_prefetch": 0}}, "positive int"),
                     ({"swap_config": {"swap": True, "layer_swap": {"layers": [0]}}}, "list of mappings"),
                     ({"swap_config": {"swap": True, "layer_swap": [{"layers": [0], "backward_prefetch": 0}]}}, "backward_prefetch")):
        with pytest.raises(ValueError, match=msg):
            check_recompute_shapes(bad)
    with pytest.raises(ValueError, match="use_seq_parallel"):
        check_compatibility({"model": {"model_config": {"fine_grain_interleave": 2}}, "parallel_config": {}})
    with pytest.raises(ValueError, match="divisible by expert_parallel"):
        check_compatibility({"model": {"model_config": {"num_experts": 6}}, "parallel_config": {"expert_parallel": 4}})
    with pytest.raises(ValueError, match="pipeline_stage > 1"):
        check_compatibility({"parallel_config": {"seq_split_num": 2}})
    check_yaml_depth_before_loading("a: {b: {c: [1, 2, {d: 3}]}}")
    deep = "a: " + "{x: " * 12 + "1" + "}" * 12
    with pytest.raises(ValueError, match="nested deeper"):
        check_yaml_depth_before_loading(deep)


def test_training_arguments_cover_the_reference_fields_and_map_to_sections():
    import re
    from mindformers_b200.trainer import TrainingArguments
    a = TrainingArguments(expert_num=8, num_experts_chosen=2, capacity_factor=1.2, aux_loss_factor=0.01, scale_sense="dynamic",
                          loss_scale_value=4096, loss_scale_window=500, micro_batch_interleave_num=2, mp_comm_recompute=False,
                          train_dataset="/data/x.jsonl", train_dataset_in_columns=["input_ids", "labels"], repeat=2,
                          keep_checkpoint_per_n_minutes=30, profile_end_step=7, hub_model_id="org/model",
                          gradient_aggregation_group=8)
    cfg = a.convert_args_to_mindformers_config()
    assert cfg["moe_config"] == dict(expert_num=8, capacity_factor=1.2, aux_loss_factor=0.01, num_experts_chosen=2)
    assert cfg["runner_wrapper"]["scale_sense"]["type"] == "DynamicLossScaleUpdateCell"
    assert cfg["runner_wrapper"]["scale_sense"]["scale_window"] == 500
    assert cfg["micro_batch_interleave_num"] == 2 and cfg["recompute_config"]["mp_comm_recompute"] is False
    assert cfg["train_dataset"]["input_columns"] == ["input_ids", "labels"] and cfg["train_dataset"]["repeat"] == 2
    ck = [c for c in cfg["callbacks"] if c["type"] == "CheckpointMonitor"][0]
    assert ck["keep_checkpoint_per_n_minutes"] == 30 and cfg["profile_stop_step"] == 7
    assert cfg["hub"]["hub_model_id"] == "org/model" and cfg["parallel_config"]["gradient_aggregation_group"] == 8
    fields = set(TrainingArguments.__dataclass_fields__)
    for name in ("max_call_depth", "gradients_mean", "enable_alltoall", "dataset_strategy", "parallel_optimizer_threshold",
                 "recompute_slice_activation", "eval_dataset_out_columns", "prediction_loss_only", "max_scale_window",
                 "auto_tune", "hub_always_push", "strategy_ckpt_save_file"):
        assert name in fields, name


def test_3d_tensor_parallel_maps_onto_tensor_and_context_parallel():
    """``use_3d_tensor_parallel`` with tp_x / tp_y / tp_z: heads over y, sequence over (cp, z, x); the sizes must
    multiply to model_parallel and sequence parallelism is rejected, as in the reference."""
    import pytest
    from mindformers_b200.core.context import build_context, resolve_3d_tensor_parallel
    par = {"data_parallel": 1, "model_parallel": 8, "context_parallel": 2}
    mc = {"use_3d_tensor_parallel": True, "tp_x": 2, "tp_y": 2, "tp_z": 2}
    out = resolve_3d_tensor_parallel(par, mc)
    assert out["model_parallel"] == 2 and out["context_parallel"] == 8
    assert par["model_parallel"] == 2 and par["context_parallel"] == 8
    assert resolve_3d_tensor_parallel(par, mc) == out                      # a second reader changes nothing
    with pytest.raises(ValueError):
        resolve_3d_tensor_parallel({"model_parallel": 8}, {"use_3d_tensor_parallel": True, "tp_x": 2, "tp_y": 2, "tp_z": 1})
    with pytest.raises(ValueError):
        resolve_3d_tensor_parallel({"model_parallel": 4, "use_seq_parallel": True},
                                   {"use_3d_tensor_parallel": True, "tp_x": 2, "tp_y": 2, "tp_z": 1})
    assert resolve_3d_tensor_parallel({"model_parallel": 4}, {"tp_x": 2}) is None
    cfg = {"use_parallel": False, "context": {"device_target": "CPU"},
           "parallel_config": {"model_parallel": 4}, "model": {"model_config": {"use_3d_tensor_parallel": True, "tp_x": 2,
                                                                                 "tp_y": 2, "tp_z": 1}}}
    ctx = build_context(cfg)
    assert ctx.tensor_parallel_3d["context_parallel"] == 2 and cfg["parallel_config"]["model_parallel"] == 2
