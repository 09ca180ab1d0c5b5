"""Prefix-tuning / P-Tuning v2: trainable key/value prefixes per layer, base model frozen
(``mindformers/pet/tuners/prefix_tuning_adapter.py``, ``ptuning2_adapter.py``). Every layer's self-attention sees
``[prefix ‖ sequence]`` keys and values; queries attend to the whole prefix and causally to the sequence."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ..ops import functional as Fn


class PrefixEncoder(nn.Module):
    """``[P]`` virtual positions → per-layer ``(K, V)`` prefixes ``[L, 2, P, kv_heads, head_dim]``; optional MLP
    re-parameterisation (``prefix_projection``)."""

    def __init__(self, num_layers: int, kv_heads: int, head_dim: int, pre_seq_len: int, prefix_projection: bool = False,
                 projection_dim: int = 128, dropout: float = 0.0, device=None, dtype=torch.float32):
        super().__init__()
        self.L, self.kv, self.hd, self.P = num_layers, kv_heads, head_dim, pre_seq_len
        out = num_layers * 2 * kv_heads * head_dim
        if prefix_projection:
            self.embedding = nn.Embedding(pre_seq_len, projection_dim, device=device, dtype=dtype)
            self.trans = nn.Sequential(nn.Linear(projection_dim, projection_dim, device=device, dtype=dtype), nn.Tanh(),
                                       nn.Linear(projection_dim, out, device=device, dtype=dtype))
        else:
            self.embedding = nn.Embedding(pre_seq_len, out, device=device, dtype=dtype)
            self.trans = None
        nn.init.normal_(self.embedding.weight, std=0.02)
        self.dropout = nn.Dropout(dropout) if dropout > 0 else None
        self.register_buffer("positions", torch.arange(pre_seq_len, device=device), persistent=False)

    def forward(self):
        x = self.embedding(self.positions)
        if self.trans is not None:
            x = self.trans(x)
        if self.dropout is not None:
            x = self.dropout(x)
        return x.view(self.P, self.L, 2, self.kv, self.hd).permute(1, 2, 0, 3, 4)


class _PrefixCore(nn.Module):
    """Stands in for a layer's core attention: prepends the layer's prefix to K and V."""

    def __init__(self, core, owner: "PrefixTuningModel", layer_index: int):
        super().__init__()
        self.core, self.layer_index = core, layer_index
        self._owner = [owner]          # not registered as a sub-module (avoids a reference cycle in .modules())
        self.scale = core.scale

    def forward(self, q, k, v, meta):
        pk, pv = self._owner[0].current[self.layer_index]
        B, S = meta.batch, meta.seq_len
        T = q.shape[0]
        nq, hd = q.shape[-2], q.shape[-1]
        q4 = q.reshape(B, S, nq, hd)
        k4 = k.reshape(B, S, -1, hd)
        v4 = v.reshape(B, S, -1, hd)
        P = pk.shape[0]
        k4 = torch.cat([pk.to(k.dtype).unsqueeze(0).expand(B, -1, -1, -1), k4], dim=1)
        v4 = torch.cat([pv.to(v.dtype).unsqueeze(0).expand(B, -1, -1, -1), v4], dim=1)
        out = Fn.attention_reference(q4, k4, v4, causal=True, scale=self.scale, q_offset=P)
        return out.reshape(T, nq * hd)


class PrefixTuningModel(nn.Module):
    """Freezes the base model and trains per-layer prefix key / value vectors that are prepended inside attention
    (reference ``pet/tuners/prefix_tuning_adapter.py``)."""

    def __init__(self, config, base_model: nn.Module):
        super().__init__()
        self.pet_config = config
        self.network = base_model
        gpt = getattr(base_model, "model", base_model)
        tcfg = gpt.config
        for p in base_model.parameters():
            p.requires_grad_(False)
        P = getattr(config, "pre_seq_len", None) or getattr(config, "prefix_token_num", 16)
        layers = gpt.decoder.layers
        first = next(base_model.parameters())
        hd = tcfg.kv_channels or tcfg.hidden_size // tcfg.num_attention_heads
        self.prefix_encoder = PrefixEncoder(len(layers), tcfg.num_query_groups or tcfg.num_attention_heads, hd, P,
                                            getattr(config, "prefix_projection", False), getattr(config, "projection_dim", 128),
                                            getattr(config, "dropout_prob", 0.0) or getattr(config, "dropout_rate", 0.0),
                                            device=first.device)
        self.current = None
        for i, layer in enumerate(layers):
            layer.self_attention.core_attention = _PrefixCore(layer.self_attention.core_attention, self, i)
            layer.self_attention.use_packed_attention = False

    def forward(self, *a, **kw):
        self.current = self.prefix_encoder()
        return self.network(*a, **kw)
