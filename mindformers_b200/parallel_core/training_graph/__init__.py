"""Training layers under the reference's ``parallel_core/training_graph`` path."""
from ...parallel.layers.gpt_model import GPTModel  # noqa: F401
from ...parallel.layers.tensor_parallel import ColumnParallelLinear, RowParallelLinear, VocabParallelEmbedding  # noqa: F401
from ...parallel.layers.transformer_layer import TransformerBlock, TransformerLayer  # noqa: F401
from ...parallel.layers.loss import CrossEntropyLoss  # noqa: F401

__all__ = ["ColumnParallelLinear", "CrossEntropyLoss", "GPTModel", "RowParallelLinear", "TransformerBlock", "TransformerLayer", "VocabParallelEmbedding"]
