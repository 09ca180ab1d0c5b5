"""The ``deepseek3`` family under its reference import path (``mindformers/models/deepseek3``). The reference picks a
``Training...`` or ``Inference...`` class by run mode; one class serves both here, so those names are aliases, and
``DeepseekV3PreTrainedModel`` is the shared base (``PreTrainedModel`` bound to this family's configuration class)."""
from ...models.families import DeepseekV3Config, DeepseekV3ForCausalLM, InferenceDeepseekV3ForCausalLM, TrainingDeepseekV3ForCausalLM  # noqa: F401
from ...models.modeling_utils import PreTrainedModel


class DeepseekV3PreTrainedModel(PreTrainedModel):
    config_class = DeepseekV3Config
    base_model_prefix = "model"


__all__ = ['DeepseekV3Config', 'DeepseekV3ForCausalLM', 'DeepseekV3PreTrainedModel', 'InferenceDeepseekV3ForCausalLM', 'TrainingDeepseekV3ForCausalLM']
