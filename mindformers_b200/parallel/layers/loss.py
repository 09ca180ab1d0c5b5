"""Masked, vocab-parallel cross-entropy.

Reference: ``training_graph/loss_func.py`` (``_LogSoftmax``/``_NLLLoss`` with hand-written backward
:35-139, ``CrossEntropyLoss`` :142-288: ``Σ(nll·mask) / (Σmask + 1e-8)`` or the (numerator, denominator)
pair for per-token loss; ``VocabParallelCrossEntropy`` :291).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ...ops import functional as Fn
from .. import parallel_state as ps


class VocabParallelCrossEntropy(nn.Module):
    """Per-token NLL from logits sharded over the vocabulary axis."""

    def forward(self, logits, labels, vocab_start=None):
        tp = ps.get_tensor_model_parallel_world_size()
        if vocab_start is None:
            vocab_start = ps.get_tensor_model_parallel_rank() * logits.shape[-1] if tp > 1 else 0
        grp = ps.get_tensor_model_parallel_group() if tp > 1 else None
        return Fn.cross_entropy(logits, labels, vocab_start, grp)


class CrossEntropyLoss(nn.Module):
    """Masked vocabulary-parallel cross-entropy (reference ``training_graph/loss_func.py:35-139``): fp32 statistics,
    returns ``sum(loss * mask) / (sum(mask) + 1e-8)`` or the ``(numerator, denominator)`` pair for pipeline /
    sequence-pipeline accumulation."""

    def __init__(self, calculate_per_token_loss: bool = False, eps: float = 1e-8):
        super().__init__()
        self.per_token = calculate_per_token_loss
        self.eps = eps
        self.nll = VocabParallelCrossEntropy()

    def forward(self, logits, labels, loss_mask, vocab_start=None):
        logits = logits.reshape(-1, logits.shape[-1])
        labels = labels.reshape(-1)
        mask = loss_mask.reshape(-1).float()
        safe = labels.clamp(min=0)
        nll = self.nll(logits, safe, vocab_start)
        num = (nll * mask).sum()
        den = mask.sum()
        if self.per_token:
            return num, den
        return num / (den + self.eps)
