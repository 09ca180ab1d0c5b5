"""Inference layers under the reference's ``parallel_core/inference`` path (the training layers serve both)."""
from ...parallel.layers.gpt_model import GPTModel  # noqa: F401
from ...parallel.layers.tensor_parallel import ColumnParallelLinear, RowParallelLinear, VocabParallelEmbedding  # noqa: F401
from ...inference.weights_utils import WeightsLoader  # noqa: F401
from ...inference.model_utils import InferModelMixin  # noqa: F401

__all__ = ["ColumnParallelLinear", "GPTModel", "InferModelMixin", "RowParallelLinear", "VocabParallelEmbedding", "WeightsLoader"]
