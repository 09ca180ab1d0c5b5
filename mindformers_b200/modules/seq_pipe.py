"""Sequence-pipeline splitting (``mindformers/modules/seq_pipe.py:21-119``): the sequence axis is cut into
``seq_split_num`` chunks that flow through the pipeline one after another; every chunk attends to the keys and values
of the chunks before it, which the attention layers keep in a per-micro-batch cache."""
from __future__ import annotations

from typing import Dict, Iterator, List

import torch


class SequenceSplit:
    """Sequence-pipeline chunking (reference ``modules/seq_pipe.py:21,64-119``): slices the sequence axis into
    ``seq_split_num`` chunks that flow through the pipeline one after the other, relying on the KV cache of the
    earlier chunks."""

    def __init__(self, seq_split_num: int, seq_dim: int = 1):
        if seq_split_num < 1:
            raise ValueError("seq_split_num must be >= 1")
        self.n, self.dim = seq_split_num, seq_dim

    def split(self, batch: Dict[str, torch.Tensor]) -> List[Dict[str, torch.Tensor]]:
        """Chunks of a batch along the sequence axis, each with ``seq_chunk`` (its index) and ``position_ids`` that
        continue across chunks."""
        S = batch["input_ids"].shape[self.dim]
        if S % self.n:
            raise ValueError(f"sequence length {S} is not divisible by seq_split_num {self.n}")
        step = S // self.n
        out = []
        for c in range(self.n):
            sl = slice(c * step, (c + 1) * step)
            part = {k: (v[:, sl] if torch.is_tensor(v) and v.dim() >= 2 and v.shape[self.dim] == S else v) for k, v in batch.items()}
            if "position_ids" not in part or part["position_ids"] is None:
                B = batch["input_ids"].shape[0]
                part["position_ids"] = torch.arange(c * step, (c + 1) * step, device=batch["input_ids"].device).unsqueeze(0).expand(B, step)
            part["seq_chunk"] = c
            out.append(part)
        return out

    def __call__(self, batch) -> Iterator[Dict[str, torch.Tensor]]:
        return iter(self.split(batch))

    @staticmethod
    def merge_losses(numerators, denominators):
        """Per-token loss over all chunks: ``sum(numerators) / sum(denominators)`` (``loss_func.py:232,286-288``)."""
        return torch.stack(list(numerators)).sum() / (torch.stack(list(denominators)).sum() + 1e-8)
