"""The ``qwen2`` family under its reference import path (``mindformers/models/qwen2``). The reference picks a
``Training...`` or ``Inference...`` class by run mode; one class serves both here, so those names are aliases, and
``Qwen2PreTrainedModel`` is the shared base (``PreTrainedModel`` bound to this family's configuration class)."""
from ...models.families import Qwen2Config, Qwen2ForCausalLM, InferenceQwen2ForCausalLM  # noqa: F401
from ...models.modeling_utils import PreTrainedModel


class Qwen2PreTrainedModel(PreTrainedModel):
    config_class = Qwen2Config
    base_model_prefix = "model"


__all__ = ['InferenceQwen2ForCausalLM', 'Qwen2Config', 'Qwen2ForCausalLM', 'Qwen2PreTrainedModel']
