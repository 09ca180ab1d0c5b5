"""Training layers under the reference's ``parallel_core/training_graph`` path: every layer, spec container and helper of
that tree, whichever file of it a script imports them from (the deep paths resolve to this module)."""
from ...parallel.layers.attention import AttnMeta, CoreAttention, CrossAttention, MLASelfAttention, MLASelfAttentionMegatron, SelfAttention  # noqa: F401
from ...parallel.layers.building_blocks import *  # noqa: F401,F403
from ...parallel.layers.building_blocks import (ApplyRotaryPosEmb, AttnMaskType, CrossAttentionSubmodules, IdentityFuncOp, IdentityOp,  # noqa: F401
                                                MLASelfAttentionSubmodules, MLASelfAttentionSubmodulesConcatenated, MLPSubmodules,
                                                MoESubmodules, MoETokenDispatcher, MultiTokenPredictionBlockSubmodules,
                                                MultiTokenPredictionLayerSubmodules, Router, SelfAttentionSubmodules, SwiGlu,
                                                TransformerBlockSubmodules, get_act_func, get_attn_mask_func, get_norm_cls)
from ...parallel.layers.dot_product_attention import (AttnMaskFill, CausalMaskGenerate, DotProductAttention, FusedScaleMaskSoftmax,  # noqa: F401
                                                      LowerTriangularMask)
from ...parallel.layers.gpt_layer_specs import (get_gpt_decoder_block_spec, get_gpt_layer_local_spec, get_gpt_layer_spec_for_config,  # noqa: F401
                                                get_gpt_mtp_block_spec, get_mlp_module_spec, get_moe_module_spec)
from ...parallel.layers.gpt_model import GPTModel, LanguageModelEmbedding  # noqa: F401
from ...parallel.layers.mlp import MLP  # noqa: F401
from ...parallel.layers.moe import GroupedMLP, MoEAlltoAllTokenDispatcher, MoELayer, SharedExpertMLP, TopKRouter  # noqa: F401
from ...parallel.layers.mtp import MultiTokenPredictionBlock, MultiTokenPredictionLayer  # noqa: F401
from ...parallel.layers.norm import FusedLayerNorm, LayerNorm, RMSNorm  # noqa: F401
from ...parallel.layers.rotary import RotaryEmbedding, YarnRotaryEmbedding, get_rope  # noqa: F401
from ...parallel.layers.tensor_parallel import (ColumnParallelBatchedLinear, ColumnParallelLinear, LinearNoTP, RowParallelBatchedLinear,  # noqa: F401
                                                RowParallelLinear, VocabParallelEmbedding)
from ...parallel.layers.transformer_layer import TransformerBlock, TransformerLayer, TransformerLayerSubmodules  # noqa: F401
from ...modules.flash_attention import FlashAttention  # noqa: F401
from ...modules.rng import CudaRNGStatesTracker, get_rng_tracker, model_parallel_manual_seed  # noqa: F401

# names the reference gives the same classes in this tree
Attention = SelfAttention
MultiLatentAttention = MLASelfAttention
BaseTransformerLayer = TransformerLayer
BaseMoELayer = MoELayer
Norm = LayerNorm
FusedNorm = RMSNorm
FusedRMSNorm = RMSNorm
YaRNScalingRotaryEmbedding = YarnRotaryEmbedding
QKVParallelLinear = ColumnParallelLinear
MergedColumnParallelLinear = ColumnParallelLinear
ReplicatedLinear = LinearNoTP
RNGStateTracer = CudaRNGStatesTracker
get_rng_tracer = get_rng_tracker
set_rng_seed = model_parallel_manual_seed
from ...parallel.layers.loss import CrossEntropyLoss, VocabParallelCrossEntropy  # noqa: F401
from ...pet.lora import ColumnParallelLinearWithLoRA, RowParallelLinearWithLoRA  # noqa: F401

SelfAttentionContiguous = SelfAttention
MLASelfAttentionConcatenated = MLASelfAttentionMegatron
get_mtp_layer_spec = get_gpt_mtp_block_spec

from torch.nn import Dropout  # noqa: E402,F401

from ...modules.activation import GELU, SiLU, get_activation  # noqa: E402,F401
from ...parallel.layers.moe import permute, unpermute  # noqa: E402,F401
from ...parallel.layers.norm import get_norm  # noqa: E402,F401

FFNGroupedGEMM = GroupedMLP
LowerTriangularMaskWithDynamic = LowerTriangularMask
Llama3RotaryEmbedding = RotaryEmbedding            # ``rope_scaling`` of the configuration selects the Llama-3 rescaling
DATA_PARALLEL_GENERATOR = "dp_rng_generator"
TENSOR_PARALLEL_GENERATOR = "tp_rng_generator"
EXPERT_PARALLEL_GENERATOR = "exp_rng_generator"
