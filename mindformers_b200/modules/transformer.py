"""Generic transformer building blocks of the legacy stack: attention, feed-forward, encoder / decoder layers and stacks.

Reference: ``mindformers/modules/transformer/transformer.py`` (``FeedForward``, ``MultiHeadAttention``,
``TransformerEncoderLayer``, ``TransformerDecoderLayer``, ``TransformerEncoder``, ``TransformerDecoder``,
``Transformer``, ``AttentionMask``, ``VocabEmbedding``; the classes that models written against the older API are
assembled from). Conventions kept from there: inputs are ``[batch, seq, hidden]``; attention masks are
``[batch, q_len, k_len]`` with 1 = may attend; ``post_layernorm_residual`` chooses between post-LN (residual taken
after the norm) and pre-LN; every layer returns ``(output, layer_present)`` where ``layer_present`` is the
``(key, value)`` pair for incremental decoding; ``parallel_config`` is accepted and only its recompute switch is used
(tensor-parallel models are built from ``parallel/layers`` instead).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from .activation import get_activation


class AttentionMask(nn.Module):
    """``input_mask [batch, seq]`` (1 = real token) → causal ``[batch, seq, seq]`` mask (1 = may attend)."""

    def __init__(self, seq_length: int, parallel_config=None):
        super().__init__()
        self.register_buffer("tril", torch.tril(torch.ones(seq_length, seq_length)), persistent=False)

    def forward(self, input_mask: torch.Tensor) -> torch.Tensor:
        S = input_mask.shape[1]
        m = input_mask.to(self.tril.dtype)
        return m[:, :, None] * m[:, None, :] * self.tril[:S, :S]


class VocabEmbedding(nn.Module):
    """Token embedding; returns ``(embeddings, table)`` so that the output head can share the table."""

    def __init__(self, vocab_size: int, embedding_size: int, parallel_config=None, param_init: float = 0.02):
        super().__init__()
        self.embedding_table = nn.Parameter(torch.empty(vocab_size, embedding_size).normal_(0, param_init))

    def forward(self, input_ids: torch.Tensor):
        return F.embedding(input_ids, self.embedding_table), self.embedding_table


class FeedForward(nn.Module):
    """``dropout(W2 act(W1 x))``."""

    def __init__(self, hidden_size: int, ffn_hidden_size: int, dropout_rate: float = 0.1, hidden_act: str = "gelu",
                 expert_num: int = 1, parallel_config=None):
        super().__init__()
        if expert_num != 1:
            raise ValueError("mixture-of-experts feed-forward layers are modules.moe_legacy.MoEV2 / MoEV3")
        self.mapping = nn.Linear(hidden_size, ffn_hidden_size)
        self.projection = nn.Linear(ffn_hidden_size, hidden_size)
        self.act = get_activation(hidden_act)
        self.dropout = nn.Dropout(dropout_rate)

    def forward(self, x):
        return self.dropout(self.projection(self.act(self.mapping(x))))


class MultiHeadAttention(nn.Module):
    """Scaled dot-product attention with separate query and key / value inputs (self- or cross-attention) and an
    optional key / value history for incremental decoding."""

    def __init__(self, batch_size: Optional[int], src_seq_length: int, tgt_seq_length: int, hidden_size: int,
                 num_heads: int, hidden_dropout_rate: float = 0.1, attention_dropout_rate: float = 0.1,
                 use_past: bool = False, parallel_config=None):
        super().__init__()
        if hidden_size % num_heads:
            raise ValueError("hidden_size must be divisible by num_heads")
        self.h, self.d = num_heads, hidden_size // num_heads
        self.dense1, self.dense2, self.dense3 = (nn.Linear(hidden_size, hidden_size) for _ in range(3))
        self.projection = nn.Linear(hidden_size, hidden_size)
        self.prob_dropout = nn.Dropout(attention_dropout_rate)
        self.dropout = nn.Dropout(hidden_dropout_rate)
        self.use_past = use_past

    def _split(self, x):
        B, S, _ = x.shape
        return x.view(B, S, self.h, self.d).transpose(1, 2)

    def forward(self, query_tensor, key_tensor, value_tensor, attention_mask=None, key_past=None, value_past=None,
                batch_valid_length=None):
        q = self._split(self.dense1(query_tensor))
        k = self._split(self.dense2(key_tensor))
        v = self._split(self.dense3(value_tensor))
        if self.use_past and key_past is not None:
            k, v = torch.cat((key_past, k), dim=2), torch.cat((value_past, v), dim=2)
        scores = torch.matmul(q, k.transpose(-1, -2)) / math.sqrt(self.d)
        if attention_mask is not None:
            scores = scores.masked_fill(attention_mask[:, None].to(torch.bool).logical_not(), -10000.0)
        probs = self.prob_dropout(torch.softmax(scores.float(), dim=-1).to(v.dtype))
        out = torch.matmul(probs, v).transpose(1, 2).reshape(query_tensor.shape[0], query_tensor.shape[1], -1)
        return self.dropout(self.projection(out)), (k, v)


class TransformerEncoderLayer(nn.Module):
    def __init__(self, batch_size: Optional[int], hidden_size: int, ffn_hidden_size: int, num_heads: int,
                 seq_length: int, attention_dropout_rate: float = 0.1, hidden_dropout_rate: float = 0.1,
                 post_layernorm_residual: bool = False, hidden_act: str = "gelu", use_past: bool = False,
                 parallel_config=None):
        """One encoder block: self-attention and feed-forward, each with a residual connection and a LayerNorm."""
        super().__init__()
        self.post = post_layernorm_residual
        self.layernorm1, self.layernorm2 = nn.LayerNorm(hidden_size), nn.LayerNorm(hidden_size)
        self.attention = MultiHeadAttention(batch_size, seq_length, seq_length, hidden_size, num_heads,
                                            hidden_dropout_rate, attention_dropout_rate, use_past, parallel_config)
        self.output = FeedForward(hidden_size, ffn_hidden_size, hidden_dropout_rate, hidden_act)

    def forward(self, x, input_mask=None, init_reset=True, batch_valid_length=None, key_past=None, value_past=None):
        normed = self.layernorm1(x)
        attn, present = self.attention(normed, normed, normed, input_mask, key_past, value_past, batch_valid_length)
        x = (normed if self.post else x) + attn
        normed = self.layernorm2(x)
        x = (normed if self.post else x) + self.output(normed)
        return x, present


class TransformerDecoderLayer(nn.Module):
    def __init__(self, hidden_size: int, ffn_hidden_size: int, num_heads: int, batch_size: Optional[int],
                 src_seq_length: int, tgt_seq_length: int, attention_dropout_rate: float = 0.1,
                 hidden_dropout_rate: float = 0.1, post_layernorm_residual: bool = False, use_past: bool = False,
                 hidden_act: str = "gelu", parallel_config=None):
        """One decoder block: masked self-attention, cross-attention over the encoder output, feed-forward."""
        super().__init__()
        self.post = post_layernorm_residual
        self.layernorm1, self.layernorm2, self.cross_attention_layernorm = (nn.LayerNorm(hidden_size) for _ in range(3))
        self.attention = MultiHeadAttention(batch_size, tgt_seq_length, tgt_seq_length, hidden_size, num_heads,
                                            hidden_dropout_rate, attention_dropout_rate, use_past, parallel_config)
        self.cross_attention = MultiHeadAttention(batch_size, tgt_seq_length, src_seq_length, hidden_size, num_heads,
                                                  hidden_dropout_rate, attention_dropout_rate, False, parallel_config)
        self.output = FeedForward(hidden_size, ffn_hidden_size, hidden_dropout_rate, hidden_act)

    def forward(self, hidden_stats, decoder_mask=None, encoder_output=None, memory_mask=None, init_reset=True,
                batch_valid_length=None, key_past=None, value_past=None):
        normed = self.layernorm1(hidden_stats)
        attn, present = self.attention(normed, normed, normed, decoder_mask, key_past, value_past, batch_valid_length)
        x = (normed if self.post else hidden_stats) + attn
        if encoder_output is not None:
            normed = self.cross_attention_layernorm(x)
            cross, _ = self.cross_attention(normed, encoder_output, encoder_output, memory_mask)
            x = (normed if self.post else x) + cross
        normed = self.layernorm2(x)
        x = (normed if self.post else x) + self.output(normed)
        return x, present


def _wants_recompute(parallel_config) -> bool:
    rc = getattr(parallel_config, "recompute", None)
    flag = getattr(rc, "recompute", rc)
    return bool(flag) if isinstance(flag, (bool, int)) else False


class TransformerEncoder(nn.Module):
    """``num_layers`` encoder blocks; returns ``(output, [layer_present, ...])``."""

    def __init__(self, batch_size: Optional[int], num_layers: int, hidden_size: int, ffn_hidden_size: int,
                 seq_length: int, num_heads: int, attention_dropout_rate: float = 0.1, hidden_dropout_rate: float = 0.1,
                 hidden_act: str = "gelu", post_layernorm_residual: bool = False, use_past: bool = False,
                 parallel_config=None, **kw):
        super().__init__()
        self.recompute = _wants_recompute(parallel_config)
        self.blocks = nn.ModuleList([
            TransformerEncoderLayer(batch_size, hidden_size, ffn_hidden_size, num_heads, seq_length,
                                    attention_dropout_rate, hidden_dropout_rate, post_layernorm_residual, hidden_act,
                                    use_past, parallel_config) for _ in range(num_layers)])

    def forward(self, hidden_states, attention_mask=None, init_reset=True, batch_valid_length=None, past=None):
        present = []
        for i, blk in enumerate(self.blocks):
            kp, vp = past[i] if past else (None, None)
            if self.recompute and self.training and kp is None:
                hidden_states, p = checkpoint(blk, hidden_states, attention_mask, use_reentrant=False)
            else:
                hidden_states, p = blk(hidden_states, attention_mask, init_reset, batch_valid_length, kp, vp)
            present.append(p)
        return hidden_states, present


class TransformerDecoder(nn.Module):
    """``num_layers`` decoder blocks over an optional encoder output; returns ``(output, [layer_present, ...])``."""

    def __init__(self, num_layers: int, batch_size: Optional[int], hidden_size: int, ffn_hidden_size: int,
                 src_seq_length: int, tgt_seq_length: int, num_heads: int, attention_dropout_rate: float = 0.1,
                 hidden_dropout_rate: float = 0.1, post_layernorm_residual: bool = False, hidden_act: str = "gelu",
                 use_past: bool = False, parallel_config=None, **kw):
        super().__init__()
        self.blocks = nn.ModuleList([
            TransformerDecoderLayer(hidden_size, ffn_hidden_size, num_heads, batch_size, src_seq_length, tgt_seq_length,
                                    attention_dropout_rate, hidden_dropout_rate, post_layernorm_residual, use_past,
                                    hidden_act, parallel_config) for _ in range(num_layers)])

    def forward(self, hidden_stats, attention_mask=None, encoder_output=None, memory_mask=None, init_reset=True,
                batch_valid_length=None, past=None):
        present = []
        for i, blk in enumerate(self.blocks):
            kp, vp = past[i] if past else (None, None)
            hidden_stats, p = blk(hidden_stats, attention_mask, encoder_output, memory_mask, init_reset,
                                  batch_valid_length, kp, vp)
            present.append(p)
        return hidden_stats, present


class Transformer(nn.Module):
    """Encoder-decoder (or encoder-only with ``decoder_layers=0``): returns
    ``(output, encoder_layer_present, decoder_layer_present)``."""

    def __init__(self, hidden_size: int, batch_size: Optional[int], ffn_hidden_size: int, src_seq_length: int,
                 tgt_seq_length: int, encoder_layers: int = 3, decoder_layers: int = 3, num_heads: int = 2,
                 attention_dropout_rate: float = 0.1, hidden_dropout_rate: float = 0.1, hidden_act: str = "gelu",
                 post_layernorm_residual: bool = False, parallel_config=None, **kw):
        super().__init__()
        if encoder_layers <= 0 and decoder_layers <= 0:
            raise ValueError("a Transformer needs encoder layers, decoder layers or both")
        self.encoder = TransformerEncoder(batch_size, encoder_layers, hidden_size, ffn_hidden_size, src_seq_length,
                                          num_heads, attention_dropout_rate, hidden_dropout_rate, hidden_act,
                                          post_layernorm_residual, False, parallel_config) if encoder_layers > 0 else None
        self.decoder = TransformerDecoder(decoder_layers, batch_size, hidden_size, ffn_hidden_size, src_seq_length,
                                          tgt_seq_length, num_heads, attention_dropout_rate, hidden_dropout_rate,
                                          post_layernorm_residual, hidden_act, False, parallel_config) \
            if decoder_layers > 0 else None

    def forward(self, encoder_inputs, encoder_masks=None, decoder_inputs=None, decoder_masks=None, memory_mask=None,
                init_reset=True, batch_valid_length=None) -> Tuple[torch.Tensor, list, Optional[list]]:
        enc_out, enc_present = (self.encoder(encoder_inputs, encoder_masks) if self.encoder is not None
                                else (encoder_inputs, []))
        if self.decoder is None:
            return enc_out, enc_present, None
        if decoder_inputs is None:
            raise ValueError("decoder_inputs are required when the Transformer has decoder layers")
        out, dec_present = self.decoder(decoder_inputs, decoder_masks, enc_out if self.encoder is not None else None,
                                        memory_mask)
        return out, enc_present, dec_present


# the parallel configuration objects live in ``core/parallel_config.py``; the reference exports them from here too
# (``modules/transformer/__init__.py``)
from ..core.parallel_config import (EmbeddingOpParallelConfig, MoEParallelConfig, OpParallelConfig,  # noqa: E402,F401
                                    TransformerOpParallelConfig, TransformerRecomputeConfig, TransformerSwapConfig)

from .._submodules import alias_children as _alias_children  # noqa: E402

_alias_children(__name__, ['transformer', 'op_parallel_config', ('moe', 'mindformers_b200.modules.moe_legacy'), ('moev3', 'mindformers_b200.modules.moe_legacy'), ('moe_utils', 'mindformers_b200.modules.moe_legacy')])
