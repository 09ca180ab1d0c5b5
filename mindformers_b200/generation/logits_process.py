"""Logits processors and warpers (device tensors).

Reference catalogue: ``generation/logits_process.py:213-685`` — temperature, repetition / frequency / presence
penalties, top-k, top-p, min-length, min-new-tokens, logit normalisation. Each is a callable
``(input_ids [B, L], scores [B, V]) -> scores``; sequences shorter than ``L`` are right-padded with ``pad``.
"""
from __future__ import annotations

from typing import Iterable, List, Optional

import torch


class LogitsProcessor:
    """Base of the score transforms: ``__call__(input_ids, scores) -> scores`` on ``[batch, vocab]`` (reference
    ``generation/logits_process.py``)."""

    def __call__(self, input_ids: torch.Tensor, scores: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class LogitsProcessorList(list):
    """Applies its processors in order."""

    def __call__(self, input_ids, scores, **kw):
        for p in self:
            scores = p(input_ids, scores)
        return scores


class TemperatureLogitsWarper(LogitsProcessor):
    """Divides the scores by ``temperature``."""

    def __init__(self, temperature: float):
        if not temperature > 0:
            raise ValueError(f"temperature must be positive, got {temperature}")
        self.t = float(temperature)

    def __call__(self, input_ids, scores):
        return scores / self.t


class RepetitionPenaltyLogitsProcessor(LogitsProcessor):
    """Scales the scores of tokens already in the sequence: positive ones divided, negative ones multiplied by
    ``repetition_penalty``."""

    def __init__(self, repetition_penalty: float):
        if not repetition_penalty > 0:
            raise ValueError("repetition_penalty must be positive")
        self.p = float(repetition_penalty)

    def __call__(self, input_ids, scores):
        ids = input_ids.clamp(min=0)
        picked = scores.gather(1, ids)
        picked = torch.where(picked < 0, picked * self.p, picked / self.p)
        valid = input_ids >= 0
        return scores.scatter(1, ids, torch.where(valid, picked, scores.gather(1, ids)))


class FrequencyPenaltyLogitsProcessor(LogitsProcessor):
    """Subtracts ``frequency_penalty`` times the number of occurrences of every token so far."""

    def __init__(self, frequency_penalty: float, output_tokens_counts: Optional[torch.Tensor] = None):
        self.p = float(frequency_penalty)

    def __call__(self, input_ids, scores):
        counts = torch.zeros_like(scores)
        ones = (input_ids >= 0).to(scores.dtype)
        counts.scatter_add_(1, input_ids.clamp(min=0), ones)
        return scores - self.p * counts


class PresencePenaltyLogitsProcessor(LogitsProcessor):
    """Subtracts ``presence_penalty`` from every token that occurred at least once."""

    def __init__(self, presence_penalty: float):
        self.p = float(presence_penalty)

    def __call__(self, input_ids, scores):
        seen = torch.zeros_like(scores)
        seen.scatter_(1, input_ids.clamp(min=0), (input_ids >= 0).to(scores.dtype))
        return scores - self.p * seen


class TopKLogitsWarper(LogitsProcessor):
    """Keeps the ``top_k`` highest scores, sets the rest to ``filter_value``."""

    def __init__(self, top_k: int, filter_value: float = -float("inf"), min_tokens_to_keep: int = 1):
        if top_k <= 0:
            raise ValueError("top_k must be a positive integer")
        self.k, self.fill = max(int(top_k), min_tokens_to_keep), filter_value

    def __call__(self, input_ids, scores):
        k = min(self.k, scores.shape[-1])
        kth = scores.topk(k, dim=-1).values[..., -1:]
        return scores.masked_fill(scores < kth, self.fill)


class TopPLogitsWarper(LogitsProcessor):
    """Nucleus filter: keeps the smallest set of tokens whose probabilities sum to ``top_p`` (at least
    ``min_tokens_to_keep``)."""

    def __init__(self, top_p: float, filter_value: float = -float("inf"), min_tokens_to_keep: int = 1):
        if not 0 <= top_p <= 1.0:
            raise ValueError("top_p must lie in [0, 1]")
        self.p, self.fill, self.keep = float(top_p), filter_value, min_tokens_to_keep

    def __call__(self, input_ids, scores):
        sorted_scores, idx = scores.sort(dim=-1, descending=True)
        cum = sorted_scores.softmax(-1).cumsum(-1)
        remove = cum - sorted_scores.softmax(-1) > self.p
        remove[..., : self.keep] = False
        mask = torch.zeros_like(remove).scatter(1, idx, remove)
        return scores.masked_fill(mask, self.fill)


class MinLengthLogitsProcessor(LogitsProcessor):
    """Forbids the end-of-sequence tokens until the sequence has ``min_length`` tokens."""

    def __init__(self, min_length: int, eos_token_id, pad_token_id: Optional[int] = None):
        self.min_length = int(min_length)
        self.eos = list(eos_token_id) if isinstance(eos_token_id, (list, tuple)) else [int(eos_token_id)]

    def __call__(self, input_ids, scores):
        lengths = (input_ids >= 0).sum(-1)
        short = lengths < self.min_length
        if short.any():
            scores = scores.clone()
            for e in self.eos:
                scores[short, e] = -float("inf")
        return scores


class MinNewTokensLengthLogitsProcessor(MinLengthLogitsProcessor):
    """Forbids the end-of-sequence tokens until ``min_new_tokens`` tokens were generated after the prompt."""

    def __init__(self, prompt_length_to_skip: int, min_new_tokens: int, eos_token_id, pad_token_id=None):
        super().__init__(prompt_length_to_skip + min_new_tokens, eos_token_id, pad_token_id)


class LogitNormalization(LogitsProcessor):
    """Replaces the scores by their log-softmax (after the other processors, so beam scores stay comparable)."""

    def __call__(self, input_ids, scores):
        return scores.log_softmax(dim=-1)


class GreedySearchLogitsProcessor(LogitsProcessor):
    """Argmax as a processor (keeps the reference's class name available)."""

    def __call__(self, input_ids, scores):
        return scores.argmax(-1)


class SamplingLogitsProcessor(LogitsProcessor):
    """Temperature → top-k → top-p in one object (``do_sample`` path)."""

    def __init__(self, do_sample=True, temperature=1.0, top_k=50, top_p=1.0, seed: Optional[int] = None):
        self.steps = LogitsProcessorList()
        if temperature and temperature != 1.0:
            self.steps.append(TemperatureLogitsWarper(temperature))
        if top_k and top_k > 0:
            self.steps.append(TopKLogitsWarper(top_k))
        if top_p is not None and top_p < 1.0:
            self.steps.append(TopPLogitsWarper(top_p))

    def __call__(self, input_ids, scores):
        return self.steps(input_ids, scores)


def build_processors(cfg, prompt_len: int) -> LogitsProcessorList:
    """Processors implied by a ``GenerationConfig`` (penalties first, then length constraints)."""
    out = LogitsProcessorList()
    if cfg.repetition_penalty and cfg.repetition_penalty != 1.0:
        out.append(RepetitionPenaltyLogitsProcessor(cfg.repetition_penalty))
    if cfg.frequency_penalty:
        out.append(FrequencyPenaltyLogitsProcessor(cfg.frequency_penalty))
    if cfg.presence_penalty:
        out.append(PresencePenaltyLogitsProcessor(cfg.presence_penalty))
    eos = cfg.eos_ids()
    if cfg.min_length and eos:
        out.append(MinLengthLogitsProcessor(cfg.min_length, eos))
    if cfg.min_new_tokens and eos:
        out.append(MinNewTokensLengthLogitsProcessor(prompt_len, cfg.min_new_tokens, eos))
    if cfg.renormalize_logits:
        out.append(LogitNormalization())
    return out
