"""Building blocks of the older ("legacy") model stack and small shared utilities: plain layers, activations, rotary
frequency managers with context-extension methods, ALiBi, capacity-based MoE, sequence-pipeline splitting, weight-only
and W8A8 quantisers, RNG tracker."""
from .activation import GELU, FastGelu, SiLU, SwiGLU, get_activation
from .infer_attention import InferAttention, KVCacheMgr, PagedAttentionMgr
from .layers import AlibiTensor, Dropout, FreqsMgr, LayerNorm, Linear, LowerTriangularMaskWithDynamic
from .local_block_sparse_attention import LocalBlockSparseAttention
from .moe_legacy import MoEConfig, MoEInfer, MoEV2, MoEV3, TopkRouterV2
from .seq_pipe import SequenceSplit
from .transformer import (AttentionMask, FeedForward, MultiHeadAttention, Transformer, TransformerDecoder,
                          TransformerDecoderLayer, TransformerEncoder, TransformerEncoderLayer, VocabEmbedding)
from .rng import CudaRNGStatesTracker, get_rng_tracker, model_parallel_manual_seed
