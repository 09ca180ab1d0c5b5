"""The ``qwen3_moe`` family under its reference import path (``mindformers/models/qwen3_moe``). The reference picks a
``Training...`` or ``Inference...`` class by run mode; one class serves both here, so those names are aliases, and
``Qwen3MoePreTrainedModel`` is the shared base (``PreTrainedModel`` bound to this family's configuration class)."""
from ...models.families import Qwen3MoeConfig, Qwen3MoeForCausalLM, InferenceQwen3MoeForCausalLM, TrainingQwen3MoeForCausalLM  # noqa: F401
from ...models.modeling_utils import PreTrainedModel


class Qwen3MoePreTrainedModel(PreTrainedModel):
    config_class = Qwen3MoeConfig
    base_model_prefix = "model"


__all__ = ['InferenceQwen3MoeForCausalLM', 'Qwen3MoeConfig', 'Qwen3MoeForCausalLM', 'Qwen3MoePreTrainedModel', 'TrainingQwen3MoeForCausalLM']
