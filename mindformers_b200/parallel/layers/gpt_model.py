"""``GPTModel``: embedding → rotary table → transformer block → (MTP) → output layer → loss.

One class serves training and inference (the reference has two: ``training_graph/base_models/gpt/
gpt_model.py:52-543`` and ``inference/base_models/gpt/gpt_model.py:63-392``). Semantics kept from the
reference: no label shift inside the model (the dataset supplies tokens and labels of equal length,
``gpt_model.py:305-307``); loss mask = ``(input_ids != pad) · (labels != ignore)`` unless given (:464-470);
MoE aux and MTP losses are added to the LM loss (:334,349); in prefill only the last token of each
sequence reaches the output layer (inference ``gpt_model.py:223-229``).

Parameter names follow the Megatron-style contract: ``embedding.word_embeddings.weight``,
``decoder.layers.{i}.…``, ``decoder.final_layernorm.weight``, ``output_layer.weight``, ``mtp.layers.{j}.…``.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .. import mappings as M
from .. import parallel_state as ps
from .attention import AttnMeta
from .loss import CrossEntropyLoss
from .rotary import get_rope
from .tensor_parallel import ColumnParallelLinear, VocabParallelEmbedding
from .transformer_layer import TransformerBlock


class LanguageModelEmbedding(nn.Module):
    """Word embedding (vocabulary-parallel), flattened to ``[tokens, hidden]``, scattered over the sequence-parallel
    ranks when those are on (reference ``base_models/common/embeddings/language_model_embedding.py:31``)."""

    def __init__(self, config):
        super().__init__()
        sp = bool(config.sequence_parallel) and ps.get_tensor_model_parallel_world_size() > 1
        self.word_embeddings = VocabParallelEmbedding(config.vocab_size, config.hidden_size, config=config,
                                                      reduce_scatter_embeddings=sp)
        self.sp = sp

    def forward(self, input_ids):
        return self.word_embeddings(input_ids)


class GPTModel(nn.Module):
    """The decoder-only model for training and inference (reference ``base_models/gpt/gpt_model.py``): embedding →
    rotary tables → ``TransformerBlock`` → optional multi-token-prediction block → output layer (tied or untied) →
    fp32 logits, or the masked cross-entropy when ``labels`` are given. ``forward(input_ids, labels=None,
    loss_mask=None, position_ids=None, attn_meta=None, input_embeds=None)``; ``update_topk_bias()`` applies the
    auxiliary-loss-free router balancing."""

    def __init__(self, config, pre_process: bool = True, post_process: bool = True, vp_stage: Optional[int] = None,
                 share_embeddings_and_output_weights: Optional[bool] = None):
        super().__init__()
        self.config = config
        self.pre_process, self.post_process = pre_process, post_process
        self.tied = (not config.untie_embeddings_and_output_weights) if share_embeddings_and_output_weights is None \
            else share_embeddings_and_output_weights
        dev = getattr(config, "device", None) or ("cuda" if torch.cuda.is_available() else "cpu")
        # every building block draws its initial weights from a generator seeded by (process seed, block): the values
        # do not depend on which other blocks this pipeline stage builds
        from ..init_method import module_rng
        seed0 = torch.initial_seed()
        if pre_process:
            with module_rng(seed0, 1, dev):
                self.embedding = LanguageModelEmbedding(config)
        self.rotary_pos_emb = get_rope(config, device=dev) if config.position_embedding_type in ("rope", "yarn", "llama3") else None
        self.decoder = TransformerBlock(config, pre_process, post_process, vp_stage, base_seed=seed0)
        if post_process:
            if config.mtp_num_layers:
                from .mtp import MultiTokenPredictionBlock
                with module_rng(seed0, 70, dev):
                    self.mtp = MultiTokenPredictionBlock(config)
            else:
                self.mtp = None
            with module_rng(seed0, 60, dev):
                self.output_layer = ColumnParallelLinear(config.hidden_size, config.vocab_size, config=config,
                                                         bias=False, gather_output=False,
                                                         skip_weight_param_allocation=self.tied and pre_process)
            self.loss = CrossEntropyLoss(config.calculate_per_token_loss)
        self.input_tensor = None  # activation received from the previous pipeline stage

    # ---------------------------------------------------------------------------------------------
    def set_input_tensor(self, t):
        self.input_tensor = t

    def shared_embedding_or_output_weight(self):
        if self.pre_process:
            return self.embedding.word_embeddings.weight
        return self.output_layer.weight

    def _output_weight(self):
        if self.tied and self.pre_process:
            return self.embedding.word_embeddings.weight
        return self.output_layer.weight

    def logits(self, hidden):
        """Vocab-sharded logits ``[T, V/tp]`` of hidden states ``[T(/tp under SP), H]``."""
        w = self._output_weight()
        y, _ = self.output_layer(hidden, weight=w)
        return y

    # ---------------------------------------------------------------------------------------------
    def forward(self, input_ids: torch.Tensor, labels: Optional[torch.Tensor] = None,
                loss_mask: Optional[torch.Tensor] = None, position_ids: Optional[torch.Tensor] = None,
                attn_meta: Optional[AttnMeta] = None, return_hidden: bool = False,
                input_embeds: Optional[torch.Tensor] = None, actual_seq_len: Optional[torch.Tensor] = None):
        """``input_ids``/``labels``: ``[B, S]``. Returns the loss when labels are given, else logits ``[T, V/tp]``.
        ``input_embeds`` ``[B, S, H]`` (full sequence on every tensor-parallel rank) replaces the embedding lookup;
        multimodal models use it to splice encoder outputs into the text embeddings."""
        cfg = self.config
        if input_ids.dim() == 1:
            input_ids = input_ids.unsqueeze(0)
        B, S = input_ids.shape
        meta = attn_meta or AttnMeta(batch=B, seq_len=S)
        if meta.seq_len == 0:
            meta.seq_len = S
        meta.batch = meta.batch or B
        if position_ids is not None and meta.positions is None:
            meta.positions = position_ids.reshape(-1)
        if actual_seq_len is not None and meta.actual_seq_len is None:
            # packed rows: cumulative document ends per row, as datasets with ``create_compressed_eod_mask`` emit them
            # (reference ``transformer_config.py:466-487`` / ``gpt_dataset.py:612-636``); attention stays inside documents
            meta.actual_seq_len = actual_seq_len
        if self.pre_process and input_embeds is not None:
            hidden = input_embeds.reshape(B * S, -1)
            if self.embedding.sp:
                hidden = M.scatter_to_sequence_parallel_region(hidden)
        elif self.pre_process:
            hidden = self.embedding(input_ids)
        else:
            hidden = self.input_tensor
        rotary = self.rotary_pos_emb() if self.rotary_pos_emb is not None else None
        hidden, aux = self.decoder(hidden, rotary, meta)
        if not self.post_process:
            return hidden if aux is None else (hidden, aux)
        if return_hidden:
            return hidden
        if labels is None:
            cache = meta.cache
            if cache is not None and getattr(cache, "is_prefill", False):
                hidden = hidden.index_select(0, cache.last_token_index)
            return self.logits(hidden).float()
        if loss_mask is None:
            loss_mask = (input_ids != cfg.pad_token_id) & (labels != cfg.ignore_token_id)
        else:
            loss_mask = loss_mask.to(torch.bool) & (labels != cfg.ignore_token_id)
        logits = self.logits(hidden)
        loss = self.loss(logits, labels, loss_mask)
        if cfg.calculate_per_token_loss:
            num, den = loss
            if aux is not None:
                num = num + aux * den
            return num, den
        if self.mtp is not None:
            mtp_loss = self.mtp(self, hidden, input_ids, labels, loss_mask, rotary, meta)
            loss = loss + mtp_loss
        if aux is not None:
            loss = loss + aux
        return loss

    @torch.no_grad()
    def update_topk_bias(self):
        """Aux-loss-free balancing step for every router that carries an expert bias."""
        grp = ps.get_data_parallel_group(with_context_parallel=True)
        for mod in self.modules():
            if hasattr(mod, "update_expert_bias"):
                mod.update_expert_bias(grp)
