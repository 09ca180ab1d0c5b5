"""Multi-token prediction head (DeepSeek-V3).

Reference: ``training_graph/transformer/multi_token_prediction.py`` (:87-448): tokens rolled left by one,
shared embedding, ``enorm``/``hnorm``, ``eh_proj`` (2H→H), one transformer layer, final norm, shared output
head, CE loss scaled by ``mtp_loss_scaling_factor / mtp_num_layers``. One MTP layer is supported
(``transformer_config.py:428-432``).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .norm import build_norm
from .tensor_parallel import LinearNoTP
from .transformer_layer import TransformerLayer


def roll_left(t: torch.Tensor, fill=0):
    out = torch.roll(t, shifts=-1, dims=-1)
    out[..., -1] = fill
    return out


class MultiTokenPredictionLayer(nn.Module):
    """One multi-token-prediction depth (reference ``training_graph/transformer/multi_token_prediction.py:87``): norms
    of the shifted embedding and the previous hidden state, ``eh_proj`` (2H → H), one transformer layer, final
    norm."""

    def __init__(self, config):
        super().__init__()
        self.enorm = build_norm(config)
        self.hnorm = build_norm(config)
        self.eh_proj = LinearNoTP(2 * config.hidden_size, config.hidden_size, config=config)
        pattern = config.moe_layer_pattern()
        self.transformer_layer = TransformerLayer(config, layer_number=config.num_layers + 1,
                                                  is_moe=bool(pattern[-1]) if pattern else False)
        self.final_layernorm = build_norm(config)

    def forward(self, emb, hidden, rotary, meta):
        x = torch.cat((self.enorm(emb), self.hnorm(hidden)), dim=-1)
        x, _ = self.eh_proj(x)
        pending, residual, aux = self.transformer_layer(x, None, rotary, meta)
        out, _ = self.final_layernorm(pending, residual)
        return out, aux


class MultiTokenPredictionBlock(nn.Module):
    """Runs the MTP layers on tokens rolled left by one per depth and returns their scaled cross-entropy
    (``mtp_loss_scaling_factor / mtp_num_layers`` each) through the shared embedding and output head."""

    def __init__(self, config):
        super().__init__()
        self.config = config
        self.layers = nn.ModuleList([MultiTokenPredictionLayer(config) for _ in range(config.mtp_num_layers)])

    def forward(self, model, hidden, input_ids, labels, loss_mask, rotary, meta):
        cfg = self.config
        scale = (cfg.mtp_loss_scaling_factor or 0.1) / max(cfg.mtp_num_layers, 1)
        total = 0.0
        ids, lab, mask = input_ids, labels, loss_mask
        for layer in self.layers:
            ids, lab, mask = roll_left(ids, cfg.pad_token_id), roll_left(lab, cfg.ignore_token_id), roll_left(mask, False)
            emb = model.embedding(ids)
            hidden, aux = layer(emb, hidden, rotary, meta)
            logits = model.logits(hidden)
            loss = model.loss(logits, lab, mask & (lab != cfg.ignore_token_id))
            if isinstance(loss, tuple):
                loss = loss[0] / (loss[1] + 1e-8)
            total = total + scale * loss
            if aux is not None:
                total = total + aux
        return total
