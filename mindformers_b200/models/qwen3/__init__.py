"""The ``qwen3`` family under its reference import path (``mindformers/models/qwen3``). The reference picks a
``Training...`` or ``Inference...`` class by run mode; one class serves both here, so those names are aliases, and
``Qwen3PreTrainedModel`` is the shared base (``PreTrainedModel`` bound to this family's configuration class)."""
from ...models.families import Qwen3Config, Qwen3ForCausalLM, InferenceQwen3ForCausalLM, TrainingQwen3ForCausalLM  # noqa: F401
from ...models.modeling_utils import PreTrainedModel


class Qwen3PreTrainedModel(PreTrainedModel):
    config_class = Qwen3Config
    base_model_prefix = "model"


__all__ = ['InferenceQwen3ForCausalLM', 'Qwen3Config', 'Qwen3ForCausalLM', 'Qwen3PreTrainedModel', 'TrainingQwen3ForCausalLM']
