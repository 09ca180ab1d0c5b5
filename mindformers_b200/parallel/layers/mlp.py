"""Dense feed-forward block: ``linear_fc1`` (gate‖up, column-parallel) → SwiGLU → ``linear_fc2`` (row-parallel).

Reference: ``training_graph/transformer/mlp.py`` (:38-167) and ``inference/transformer/mlp.py`` (:126-147).
The fc1 rows are ``[gate; up]``, each half sharded over tensor-parallel ranks.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...ops import functional as Fn
from .tensor_parallel import ColumnParallelLinear, RowParallelLinear

_ACT = {"gelu": F.gelu, "silu": F.silu, "swiglu": F.silu, "relu": F.relu,
        "fast_gelu": lambda x: F.gelu(x, approximate="tanh"), "gelu_tanh": lambda x: F.gelu(x, approximate="tanh")}


def get_activation(name: str):
    key = (name or "silu").lower()
    if key not in _ACT:
        raise ValueError(f"unknown activation {name!r}")
    return _ACT[key]


class MLP(nn.Module):
    """Gated MLP: ``linear_fc1`` (column-parallel, gate and up projections fused) → SwiGLU → ``linear_fc2``
    (row-parallel; reduce-scatter under sequence parallelism). Returns ``(output, bias)`` (reference
    ``training_graph/transformer/mlp.py:38,127-167``)."""

    def __init__(self, config, ffn_hidden_size=None, is_expert: bool = False, input_size=None):
        super().__init__()
        self.config = config
        F_ = ffn_hidden_size or config.ffn_hidden_size
        H = input_size or config.hidden_size
        self.gated = config.gated_linear_unit
        self.act_name = (config.hidden_act or config.activation_func or "silu").lower()
        width = 2 * F_ if self.gated else F_
        self.linear_fc1 = ColumnParallelLinear(H, width, config=config, bias=config.add_bias_linear,
                                               partition_sections=(F_, F_) if self.gated else None,
                                               is_expert=is_expert)
        self.linear_fc2 = RowParallelLinear(F_, H, config=config, bias=config.add_bias_linear,
                                            is_expert=is_expert)

    def forward(self, hidden):
        x, _ = self.linear_fc1(hidden)
        if self.gated and self.act_name in ("silu", "swiglu"):
            x = Fn.swiglu(x)
        elif self.gated:
            g, u = x.chunk(2, dim=-1)
            x = get_activation(self.act_name)(g) * u
        else:
            x = get_activation(self.act_name)(x)
        out, bias = self.linear_fc2(x)
        return out, bias
