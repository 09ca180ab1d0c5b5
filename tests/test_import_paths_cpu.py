"""Scripts written against the reference import their classes from its module paths: those paths resolve here too."""
import importlib

import pytest

PATHS = {
    "mindformers.auto_class": ["AutoModel", "AutoTokenizer"],
    "mindformers.models.base_config": ["BaseConfig"],
    "mindformers.models.base_model": ["BaseModel"],
    "mindformers.models.build_config": ["build_model_config"],
    "mindformers.models.build_model": ["build_model", "build_network"],
    "mindformers.models.build_tokenizer": ["build_tokenizer"],
    "mindformers.models.build_processor": ["build_processor"],
    "mindformers.models.convert_slow_tokenizer": ["convert_slow_tokenizer"],
    "mindformers.models.image_processing_utils": ["BaseImageProcessor"],
    "mindformers.models.tokenization_utils_base": ["PreTrainedTokenizerBase", "BatchEncoding"],
    "mindformers.models.tokenization_utils_fast": ["PreTrainedTokenizerFast"],
    "mindformers.models.llama": ["LlamaConfig", "LlamaForCausalLM", "LlamaTokenizer", "LlamaTokenizerFast", "LlamaProcessor"],
    "mindformers.models.llama.llama_config": ["LlamaConfig"],
    "mindformers.models.llama.llama": ["LlamaForCausalLM"],
    "mindformers.models.glm2": ["ChatGLM2Config", "ChatGLM2ForConditionalGeneration", "ChatGLM4Tokenizer"],
    "mindformers.models.qwen2": ["Qwen2Config", "Qwen2ForCausalLM"],
    "mindformers.models.qwen3": ["Qwen3Config", "Qwen3ForCausalLM"],
    "mindformers.models.qwen3_moe": ["Qwen3MoeConfig", "Qwen3MoeForCausalLM"],
    "mindformers.models.deepseek3": ["DeepseekV3Config", "DeepseekV3ForCausalLM"],
    "mindformers.modules.block_tables": ["BlockTables"],
    "mindformers.modules.cache_engine": ["BlockMemPool", "CacheEngine"],
    "mindformers.modules.kvcache_mgr": ["KVCacheMgr"],
    "mindformers.modules.paged_attention_mgr": ["PagedAttentionMgr"],
    "mindformers.parallel_core.transformer_config": ["TransformerConfig"],
    "mindformers.parallel_core.model_parallel_config": ["ModelParallelConfig"],
    "mindformers.parallel_core.mf_model_config": ["MFModelConfig"],
    "mindformers.parallel_core.transformer_config_utils": ["convert_to_transformer_config"],
    "mindformers.parallel_core.process_group_config": ["ModelCommProcessGroups"],
    "mindformers.parallel_core.utils.spec_utils": ["ModuleSpec", "build_module"],
    "mindformers.parallel_core.utils.init_method": ["init_method_normal", "scaled_init_method_normal"],
    "mindformers.parallel_core.training_graph": ["GPTModel", "ColumnParallelLinear", "RowParallelLinear"],
    "mindformers.parallel_core.inference": ["GPTModel", "WeightsLoader"],
    "mindformers.parallel_core.inference.parallel_state": ["initialize_model_parallel"],
    "mindformers.pet.constants": ["PetType"],
    "mindformers.pet.models": ["LoraModel"],
    "mindformers.pet.tuners": ["LoraAdapter"],
    "mindformers.pipeline.base_pipeline": ["BasePipeline"],
    "mindformers.pipeline.pipeline": ["pipeline"],
    "mindformers.pipeline.build_pipeline": ["build_pipeline"],
    "mindformers.pipeline.text_generation_pipeline": ["TextGenerationPipeline"],
    "mindformers.trainer.build_trainer": ["build_trainer"],
    "mindformers.trainer.causal_language_modeling": ["CausalLanguageModelingTrainer"],
    "mindformers.trainer.general_task_trainer": ["GeneralTaskTrainer"],
    "mindformers.trainer.multi_modal_to_text_generation": ["MultiModalToTextGenerationTrainer"],
    "mindformers.utils.load_checkpoint_utils": ["load_checkpoint", "is_hf_safetensors_dir"],
    "mindformers.utils.resume_ckpt_utils": ["load_resume_context_from_checkpoint", "get_resume_checkpoint"],
    "mindformers.utils.quantization_config": ["RtnConfig", "PtqConfig", "SmoothQuantConfig"],
    "mindformers.wrapper.wrapper": ["MFTrainOneStepCell", "MFPipelineWithLossScaleCell"],
    "mindformers.wrapper.adaptive_loss_scale": ["AdaptiveLossScaleUpdateCell"],
    "mindformers.wrapper.build_wrapper": ["build_wrapper"],
    "mindformers.dataset.build_dataset": ["build_dataset"],
    "mindformers.dataset.dataloader": ["SFTDataLoader", "CommonDataLoader"],
    "mindformers.dataset.handler": ["AlpacaInstructDataHandler", "PackingHandler"],
    "mindformers.dataset.blended_datasets": ["GPTDataset", "IndexedDataset"],
    "mindformers.dataset.keyword_gen_dataset": ["KeyWordGenDataset"],
    "mindformers.dataset.multi_turn_dataset": ["MultiTurnDataset"],
    "mindformers.generation.utils": ["softmax", "topk"],
    "mindformers.tools.resume_ckpt": ["get_resume_checkpoint"],
    "mindformers.tools.transform_ckpt": ["main"],
    "mindformers.tools.ckpt_transform": ["TransformCkpt"],
    "mindformers.core.callback": ["MFLossMonitor", "CheckpointMonitor"],
    "mindformers.core.optim": ["AdamW", "FusedAdamW"],
    "mindformers.core.lr": ["CosineWithWarmUpLR"],
    "mindformers.core.context": ["build_context"],
}


@pytest.mark.parametrize("module", sorted(PATHS))
def test_reference_import_path_resolves(module):
    mod = importlib.import_module(module)
    for name in PATHS[module]:
        assert hasattr(mod, name), (module, name)


def test_shims_are_the_same_objects_and_builders_work():
    import numpy as np
    from mindformers.models.llama import LlamaConfig as A
    from mindformers_b200.models import LlamaConfig as B
    assert A is B
    from mindformers.pipeline.build_pipeline import build_pipeline
    from mindformers.wrapper.build_wrapper import build_wrapper
    assert build_pipeline() is None and build_wrapper() is None
    from mindformers.generation.utils import log_softmax, softmax, topk
    x = np.array([[1.0, 3.0, 2.0]])
    assert abs(softmax(x).sum() - 1) < 1e-12 and np.allclose(np.exp(log_softmax(x)), softmax(x))
    v, i = topk(x, 2)
    assert v.tolist() == [[3.0, 2.0]] and i.tolist() == [[1, 2]]


def test_function_names_survive_importing_their_modules():
    """``models.build_processor`` is a function and also a module path of the reference; importing the module (under
    either package name) must not replace the function."""
    import mindformers_b200.dataset as ds
    import mindformers_b200.models as models
    import mindformers_b200.pipeline as pl
    import mindformers_b200.trainer as tr
    for name in ("mindformers.models.build_processor", "mindformers_b200.models.build_model", "mindformers.models.build_tokenizer",
                 "mindformers.models.convert_slow_tokenizer", "mindformers.pipeline.pipeline", "mindformers.trainer.build_trainer",
                 "mindformers_b200.dataset.build_dataset", "mindformers.dataset.transforms.build_transforms"):
        mod = importlib.import_module(name)
        assert callable(getattr(mod, name.rsplit(".", 1)[1]))
    for fn in (models.build_processor, models.build_model, models.build_tokenizer, models.convert_slow_tokenizer,
               pl.pipeline, tr.build_trainer, ds.build_dataset, ds.transforms.build_transforms):
        assert callable(fn) and not isinstance(fn, type(importlib))


CHILD_PATHS = {
    "mindformers.core.callback.callback": ["MFLossMonitor", "CheckpointMonitor"],
    "mindformers.core.callback.build_callback": ["build_callback"],
    "mindformers.core.context.build_context": ["build_context"],
    "mindformers.core.loss.loss": ["CrossEntropyLoss"],
    "mindformers.core.lr.lr_schedule": ["CosineWithWarmUpLR"],
    "mindformers.core.lr.build_lr": ["build_lr"],
    "mindformers.core.metric.metric": ["PerplexityMetric"],
    "mindformers.core.optim.adamw": ["AdamW"],
    "mindformers.core.optim.came": ["CAME"],
    "mindformers.core.optim.build_optim": ["build_optim"],
    "mindformers.modules.transformer.transformer": ["TransformerOpParallelConfig", "EmbeddingOpParallelConfig"],
    "mindformers.modules.transformer.op_parallel_config": ["OpParallelConfig"],
    "mindformers.modules.transformer.moe": ["MoEConfig"],
    "mindformers.modules.quantizers.rtn_quantizer": ["AutoQuantizer"],
    "mindformers.dataset.sampler.build_sampler": ["build_sampler"],
    "mindformers.dataset.utils": ["check_dataset_config"],
    "mindformers.tools.ckpt_transform.utils": ["is_power_of_two", "make_soft_link"],
    "mindformers.generation.parallel_decoding_mcore": ["la_pre_process"],
    "mindformers.modules.flash_attention": ["FlashAttention"],
}


@pytest.mark.parametrize("path", sorted(CHILD_PATHS))
def test_reference_paths_below_single_file_modules(path):
    mod = importlib.import_module(path)
    for name in CHILD_PATHS[path]:
        assert hasattr(mod, name), f"{path} lacks {name}"
    import mindformers_b200.core.context as ctx
    assert callable(ctx.build_context) and not isinstance(ctx.build_context, type(importlib))


def _table():
    from mindformers_b200._reference_paths import PATHS
    return PATHS


@pytest.mark.parametrize("rel", sorted(_table()))
def test_reference_leaf_paths_resolve_to_their_module(rel):
    mod = importlib.import_module("mindformers." + rel)
    assert mod is importlib.import_module("mindformers_b200." + _table()[rel])
    assert importlib.import_module("mindformers_b200." + rel) is mod


def test_deep_reference_imports():
    from mindformers.dataset.blended_datasets.utils import Split, get_blend_from_list, normalize
    from mindformers.dataset.dataloader.sft_dataloader import SFTDataLoader  # noqa: F401
    from mindformers.models.auto.tokenization_auto import AutoTokenizer, tokenizer_class_from_name
    from mindformers.models.qwen3.modeling_qwen3_infer import InferenceQwen3ForCausalLM
    from mindformers.models.qwen3.utils import Qwen3PreTrainedModel
    from mindformers.parallel_core.inference.tensor_parallel.mappings import ReduceFromModelParallelRegion
    from mindformers.parallel_core.inference.transformer.moe.router import Router, TopKRouter
    from mindformers.parallel_core.training_graph.transformer.identity_op import IdentityOp
    from mindformers.parallel_core.training_graph.transformer.norm import FusedNorm, get_norm_cls
    from mindformers.pet.models.slora import SLoraModel  # noqa: F401
    from mindformers.pipeline.pipeline_registry import PipelineRegistry
    import mindformers_b200 as mf
    import torch
    assert InferenceQwen3ForCausalLM is mf.Qwen3ForCausalLM and Qwen3PreTrainedModel.config_class is mf.Qwen3Config
    assert tokenizer_class_from_name("LlamaTokenizer") is mf.LlamaTokenizer and AutoTokenizer is mf.AutoTokenizer
    assert get_blend_from_list(["30", "a", "70", "b"]) == (["a", "b"], [30.0, 70.0])
    assert get_blend_from_list(["a", "b", "c"]) == (["a", "b", "c"], None) and get_blend_from_list(["a", "b"]) == (["a", "b"], None)
    assert normalize([1, 3]) == [0.25, 0.75] and Split.valid.value == 1
    x = torch.randn(3, 4)
    assert IdentityOp()(x) is x and ReduceFromModelParallelRegion()(x) is x
    assert get_norm_cls("RMSNorm") is FusedNorm and issubclass(TopKRouter, torch.nn.Module) and Router is not None
    reg = PipelineRegistry({"text_generation": {"impl": mf.TextGenerationPipeline, "ms": ()}}, {"text-generation": "text_generation"})
    assert reg.check_task("text-generation")[0] == "text_generation" and "text_generation" in reg.get_supported_tasks()
    with pytest.raises(KeyError):
        reg.check_task("translation")
    with pytest.raises(ImportError):
        importlib.import_module("mindformers.dataset.dataloader.ms_ds_convertor")


def test_split_matrix_and_building_blocks():
    import torch
    from mindformers.dataset.blended_datasets.blended_megatron_dataset_config import convert_split_vector_to_split_matrix
    from mindformers.parallel_core.training_graph.base_models.common.embeddings.rope_utils import ApplyRotaryPosEmb
    from mindformers.parallel_core.training_graph.transformer.utils import get_attn_mask_func
    from mindformers.parallel_core.inference.transformer.activation import get_act_func
    m = convert_split_vector_to_split_matrix([0.9, 0.1, 0.0])
    assert m[2] is None and m[0][0] == 0.0 and abs(m[0][1] - 0.9) < 1e-12 and abs(m[1][1] - 1.0) < 1e-12
    both = convert_split_vector_to_split_matrix([0.9, 0.1, 0.0], [0.5, 0.5, 0.0])
    assert both[0] == (0.0, 0.5) and abs(both[1][0] - 0.9) < 1e-12
    scores, mask = torch.zeros(2, 2), torch.tensor([[0, 1], [0, 0]])
    assert get_attn_mask_func("attn_mask_fill")(scores, mask)[0, 1] == -10000 and get_attn_mask_func("attn_mask_add")(scores, mask)[0, 0] == 0
    x = torch.randn(4, 6)
    assert torch.allclose(get_act_func("swiglu")(x), torch.nn.functional.silu(x[:, :3]) * x[:, 3:], atol=1e-6)
    assert torch.allclose(get_act_func("squared_relu")(x), torch.relu(x) ** 2)
    # rotary: angles in the "halves" layout [f, f]; position 0 is the identity, norms are kept
    S, B, H, D = 5, 2, 3, 8
    inv = 1.0 / (10000 ** (torch.arange(0, D, 2).float() / D))
    f = torch.outer(torch.arange(S).float(), inv)
    freqs = torch.cat([f, f], -1).view(S, 1, 1, D)
    t = torch.randn(S, B, H, D)
    out = ApplyRotaryPosEmb()(t, freqs)
    assert torch.allclose(out[0], t[0], atol=1e-6) and torch.allclose(out.norm(dim=-1), t.norm(dim=-1), atol=1e-5)
    a, b = t[..., : D // 2], t[..., D // 2:]
    want = torch.cat([a * f.cos()[:, None, None] - b * f.sin()[:, None, None], b * f.cos()[:, None, None] + a * f.sin()[:, None, None]], -1)
    assert torch.allclose(out, want, atol=1e-5)
