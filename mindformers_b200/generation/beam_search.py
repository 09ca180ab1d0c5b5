"""Beam hypotheses bookkeeping (reference ``generation/beam_search.py``: ``BeamSearchScorer``)."""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch


class BeamHypotheses:
    """The ``num_beams`` best finished hypotheses of one batch entry, scored by length-penalised log-probability."""

    def __init__(self, num_beams: int, length_penalty: float, early_stopping: bool):
        self.num_beams, self.length_penalty, self.early_stopping = num_beams, length_penalty, early_stopping
        self.beams: List[Tuple[float, List[int]]] = []
        self.worst = 1e9

    def add(self, tokens: List[int], sum_logprobs: float, prompt_len: int):
        score = sum_logprobs / (max(len(tokens) - prompt_len, 1) ** self.length_penalty)
        if len(self.beams) < self.num_beams or score > self.worst:
            self.beams.append((score, tokens))
            if len(self.beams) > self.num_beams:
                self.beams.sort(key=lambda x: x[0])
                self.beams.pop(0)
            self.worst = min(s for s, _ in self.beams)

    def is_done(self, best_sum_logprobs: float, cur_len: int, prompt_len: int) -> bool:
        if len(self.beams) < self.num_beams:
            return False
        if self.early_stopping:
            return True
        return self.worst >= best_sum_logprobs / (max(cur_len - prompt_len, 1) ** self.length_penalty)


class BeamSearchScorer:
    """Beam bookkeeping of ``generate(num_beams > 1)`` (reference ``generation/beam_search.py``): picks the next beams
    from the top ``2 * num_beams`` candidates, moves finished ones into ``BeamHypotheses`` and finalises the best
    sequence per batch entry."""

    def __init__(self, batch_size: int, num_beams: int, length_penalty: float = 1.0, early_stopping: bool = False,
                 num_beam_hyps_to_keep: int = 1):
        self.batch_size, self.num_beams, self.keep = batch_size, num_beams, num_beam_hyps_to_keep
        self.hyps = [BeamHypotheses(num_beams, length_penalty, early_stopping) for _ in range(batch_size)]
        self.done = [False] * batch_size

    @property
    def is_done(self) -> bool:
        return all(self.done)

    def process(self, sequences: List[List[List[int]]], next_scores: torch.Tensor, next_tokens: torch.Tensor,
                next_indices: torch.Tensor, eos_ids: List[int], prompt_len: int, pad_id: int):
        """One step for all batches: returns (beam_scores, beam_tokens, beam_indices) each [B, num_beams]."""
        B, nb = self.batch_size, self.num_beams
        out_s = torch.zeros(B, nb)
        out_t = torch.full((B, nb), pad_id, dtype=torch.long)
        out_i = torch.zeros(B, nb, dtype=torch.long)
        for b in range(B):
            if self.done[b]:
                continue
            k = 0
            for rank_, (s, t, i) in enumerate(zip(next_scores[b].tolist(), next_tokens[b].tolist(), next_indices[b].tolist())):
                if t in eos_ids:
                    if rank_ >= nb:
                        continue
                    self.hyps[b].add(sequences[b][i] + [t], s, prompt_len)
                else:
                    out_s[b, k], out_t[b, k], out_i[b, k] = s, t, i
                    k += 1
                if k == nb:
                    break
            cur_len = len(sequences[b][0]) + 1
            self.done[b] = self.hyps[b].is_done(next_scores[b].max().item(), cur_len, prompt_len)
        return out_s, out_t, out_i

    def finalize(self, sequences: List[List[List[int]]], beam_scores: torch.Tensor, prompt_len: int) -> List[List[List[int]]]:
        out = []
        for b in range(self.batch_size):
            if not self.done[b] or len(self.hyps[b].beams) < self.keep:
                for k in range(self.num_beams):
                    self.hyps[b].add(sequences[b][k], beam_scores[b, k].item(), prompt_len)
            best = sorted(self.hyps[b].beams, key=lambda x: -x[0])[: self.keep]
            out.append([t for _, t in best])
        return out
