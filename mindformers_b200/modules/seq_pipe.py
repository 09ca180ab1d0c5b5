"""Sequence-pipeline splitting (``mindformers/modules/seq_pipe.py:21-119``): the sequence axis is cut into
``seq_split_num`` chunks that flow through the pipeline one after another; every chunk attends to the keys and values
of the chunks before it, which the attention layers keep in a per-micro-batch cache."""
from __future__ import annotations

from typing import Dict, Iterator, List, Optional, Tuple

import torch


class KVCarry:
    """Keys and values of the earlier sequence chunks of ONE micro-batch on ONE pipeline stage, per attention layer.

    The forward of chunk ``c`` appends its own (rotated) ``k`` / ``v`` — tensors inside that chunk's autograd graph —
    and attends to the concatenation of the *leaves* recorded for chunks ``< c`` (detached copies that require grad)
    with its own. Chunks run backward in reverse order: the backward of chunk ``c`` leaves ``dK`` / ``dV`` of the earlier
    chunks in the ``.grad`` of their leaves, and when chunk ``c' < c`` runs backward those gradients enter its graph
    together with the gradient of its output (``roots_and_grads``)."""

    def __init__(self):
        self.layers: Dict[int, List[Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]]] = {}
        self.chunk = 0
        self.start = 0          # tokens of this micro-batch row already processed (per sequence)

    def begin_chunk(self, chunk: int, start: int):
        self.chunk, self.start = chunk, start

    def extend(self, layer: int, k: torch.Tensor, v: torch.Tensor):
        """``k`` / ``v`` ``[B, S_chunk, heads, d]`` of the current chunk → ``(k_all, v_all)`` over chunks ``<= chunk``."""
        rows = self.layers.setdefault(layer, [])
        prev_k = [r[2] for r in rows[:self.chunk]]
        prev_v = [r[3] for r in rows[:self.chunk]]
        if torch.is_grad_enabled():
            rows.append((k, v, k.detach().requires_grad_(), v.detach().requires_grad_()))
        else:
            rows.append((k, v, k.detach(), v.detach()))
        if not prev_k:
            return k, v
        return torch.cat(prev_k + [k], dim=1), torch.cat(prev_v + [v], dim=1)

    def roots_and_grads(self, chunk: int):
        """Graph tensors of ``chunk`` that later chunks read, with the gradients those chunks left for them."""
        roots, grads = [], []
        for rows in self.layers.values():
            k, v, kl, vl = rows[chunk]
            for t, leaf in ((k, kl), (v, vl)):
                if leaf.grad is not None and t.requires_grad:
                    roots.append(t)
                    grads.append(leaf.grad)
        return roots, grads

    def release(self, chunk: int):
        """Drop the tensors of ``chunk`` once it has run backward (every later chunk has run backward before it)."""
        for rows in self.layers.values():
            rows[chunk] = (None, None, None, None)


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
