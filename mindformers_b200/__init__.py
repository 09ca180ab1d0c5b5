"""mindformers_b200: Blackwell-native large-model training and inference with the MindFormers API surface.

The names a user of the reference imports from the package root resolve here too; they are imported on first access so
that ``import mindformers_b200`` stays cheap (no torch extension is loaded until something needs it).
"""
from __future__ import annotations

import importlib

__version__ = "0.2.0"

_EXPORTS = {
    # models
    "AutoConfig": "models", "AutoModel": "models", "AutoModelForCausalLM": "models", "AutoTokenizer": "models",
    "AutoProcessor": "models", "PretrainedConfig": "models", "PreTrainedModel": "models",
    "PreTrainedTokenizer": "models", "LlamaConfig": "models", "LlamaForCausalLM": "models", "LlamaTokenizer": "models",
    "LlamaTokenizerFast": "models", "ChatGLM3Tokenizer": "models", "ChatGLM4Tokenizer": "models",
    "ChatGLM2ForConditionalGeneration": "models", "Qwen2Tokenizer": "models", "Llama3Tokenizer": "models",
    "build_network": "models", "build_tokenizer": "models", "build_processor": "models",
    # trainer / pipeline / generation
    "Trainer": "trainer", "TrainingArguments": "trainer", "ConfigArguments": "trainer", "TrainingEngine": "trainer",
    "pipeline": "pipeline", "TextGenerationPipeline": "pipeline", "MultiModalToTextPipeline": "pipeline",
    "GenerationConfig": "generation", "GenerationMixin": "generation", "TextStreamer": "generation",
    # registry / config
    "MindFormerConfig": "tools.register", "MindFormerRegister": "tools.register",
    "MindFormerModuleType": "tools.register",
    # runtime
    "ModelRunner": "model_runner", "run_check": "run_check", "MindFormerBook": "mindformer_book",
    "build_context": "core.context", "init_context": "core.context", "set_context": "core.context",
    "get_context": "core.context",
    # data
    "CausalLanguageModelDataset": "dataset", "KeyWordGenDataset": "dataset", "MultiTurnDataset": "dataset",
    "build_dataset": "dataset",
    # PEFT
    "LoraConfig": "pet", "LoraModel": "pet", "PetConfig": "pet", "get_pet_model": "pet",
    # wrappers
    "MFTrainOneStepCell": "wrapper", "MFPipelineWithLossScaleCell": "wrapper",
}

__all__ = sorted(_EXPORTS) + ["__version__"]

# Every other public name of these modules is reachable from the package root as well (the reference's root package
# re-exports its sub-packages wholesale, ``mindformers/__init__.py:20-245``); they are searched in this order on first use.
_SEARCH = ("core.callback", "core.lr", "core.optim", "core.loss", "core.metric", "core.clip_grad", "core.loss_scale",
           "core.parallel_config", "core.context", "dataset", "dataset.dataloaders", "dataset.handlers",
           "dataset.causal_language_model_dataset", "dataset.transforms", "dataset.sampler", "dataset.base_dataset",
           "dataset.dataloader", "generation", "generation.logits_process", "models", "models.base_config",
           "models.tokenization_utils_base", "models.auto", "models.families", "models.base_processor",
           "models.image_processing_utils", "models.multi_modal", "models.processing_utils", "models.tokenizers",
           "models.tokenization_utils", "modules", "modules.layers", "modules.transformer", "modules.activation",
           "modules.local_block_sparse_attention", "modules.moe_legacy", "pet", "pet.adapters", "pipeline", "trainer",
           "trainer.base_trainer", "tools.register", "tools.register.config", "tools.logger", "tools.utils", "wrapper",
           "utils", "model_runner", "_root_aliases")
_SUBPACKAGES = ("core", "dataset", "generation", "models", "modules", "pet", "pipeline", "trainer", "tools", "wrapper", "utils",
                "model_runner", "inference", "parallel", "checkpoint", "serving", "fault", "ops")


def _search(name: str):
    for mod in _SEARCH:
        try:
            module = importlib.import_module(f"{__name__}.{mod}")
        except ImportError:
            continue
        if name in getattr(module, "__dict__", {}) and not name.startswith("_"):
            return getattr(module, name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def __getattr__(name: str):
    mod = _EXPORTS.get(name)
    if mod is None:
        if name in _SUBPACKAGES:
            return importlib.import_module(f"{__name__}.{name}")
        value = _search(name)
        globals()[name] = value
        return value
    module = importlib.import_module(f"{__name__}.{mod}")
    if mod == name:
        return module          # the sub-package of the same name is callable and stands for the function too
    value = getattr(module, name)
    globals()[name] = value
    return value


def __dir__():
    return __all__

from ._reference_paths import PATHS as _REFERENCE_PATHS  # noqa: E402
from ._submodules import register_paths as _register_paths  # noqa: E402

_register_paths(__name__, _REFERENCE_PATHS)
