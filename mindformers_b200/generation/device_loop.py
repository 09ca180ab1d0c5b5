"""Decode loop without host work per token.

The reference's ``generate`` (``generation/text_generator.py:1017-1111``) returns to Python after every decode step
to pick the next token, extend the block tables and build the next step's inputs. Here one kernel
(``ops/csrc/decode_loop.cu``) does that on the device at the end of the step, so the forward pass and the selection
are captured together in one CUDA graph and a burst of steps is a burst of graph replays; the host reads the chosen
tokens back once per burst. The blocks of the paged KV cache are reserved for the whole generation up front, which is
what makes the block table a constant of the graph.

The fast path covers greedy decoding and plain temperature sampling (Gumbel-max: an exact sample of
``softmax(logits / T)``). Logits processors that need the token history, top-k / top-p warping, beam search and the
speculative plug-ins keep the host loop.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..ops import _lib

MAX_EOS = 8


@dataclass
class DecodeState:
    """Static device tensors that the captured step reads and the advance kernel updates in place."""

    tok: torch.Tensor        # [1, B] int64
    pos: torch.Tensor        # [B] int64
    lens: torch.Tensor       # [B] int32
    slots: torch.Tensor      # [B] int32
    table: torch.Tensor      # [B, width] int32
    hist: torch.Tensor       # [B, cap] int32
    count: torch.Tensor      # [B] int32
    finished: torch.Tensor   # [B] int32
    limit: torch.Tensor      # [B] int32
    params: torch.Tensor     # [12] int32: end-of-sequence ids (8, -1 unused), inverse temperature (float bits), seed
    block_size: int

    @classmethod
    def allocate(cls, batch: int, width: int, block_size: int, cap: int, device) -> "DecodeState":
        z = lambda *shape, dt=torch.int32: torch.zeros(*shape, dtype=dt, device=device)
        return cls(tok=z(1, batch, dt=torch.int64), pos=z(batch, dt=torch.int64), lens=torch.ones(batch, dtype=torch.int32, device=device),
                   slots=z(batch), table=z(batch, width), hist=z(batch, cap), count=z(batch), finished=z(batch),
                   limit=z(batch), params=torch.full((12,), -1, dtype=torch.int32, device=device), block_size=block_size)

    def set_sampling(self, eos: Sequence[int] = (), temperature: float = 0.0, seed: int = 0):
        """End-of-sequence ids, temperature (0: greedy) and the seed of the steps that follow. The kernel reads them from
        device memory, so a captured step serves every setting."""
        eos = [int(e) for e in eos][:MAX_EOS]
        inv_temp = 0.0 if not temperature or temperature <= 0 else 1.0 / float(temperature)
        words = np.full(12, -1, dtype=np.int32)
        words[: len(eos)] = eos
        words[8] = np.float32(inv_temp).view(np.int32)
        words[9] = 0
        words[10:12] = np.array([int(seed) & (2 ** 64 - 1)], dtype=np.uint64).view(np.int32)
        self.params.copy_(torch.from_numpy(words), non_blocking=True)

    def load(self, tokens: Sequence[int], positions: Sequence[int], table: np.ndarray, slots: np.ndarray,
             finished: Sequence[bool], limits: Sequence[int]):
        """Host values of the step that follows the prefill (one pinned staging buffer would save nothing: this runs
        once per ``generate`` call)."""
        dev = self.pos.device
        self.tok[0].copy_(torch.tensor(list(tokens), dtype=torch.int64), non_blocking=True)
        self.pos.copy_(torch.tensor(list(positions), dtype=torch.int64), non_blocking=True)
        self.lens.copy_(torch.tensor([p + 1 for p in positions], dtype=torch.int32), non_blocking=True)
        self.slots.copy_(torch.from_numpy(np.ascontiguousarray(slots, dtype=np.int32)), non_blocking=True)
        self.table.copy_(torch.from_numpy(np.ascontiguousarray(table, dtype=np.int32)), non_blocking=True)
        self.finished.copy_(torch.tensor([1 if f else 0 for f in finished], dtype=torch.int32), non_blocking=True)
        self.limit.copy_(torch.tensor(list(limits), dtype=torch.int32), non_blocking=True)
        self.count.zero_()
        del dev


def _advance_reference(logits: torch.Tensor, st: DecodeState):
    """Plain PyTorch body of ``decode_advance`` (CPU tensors; the oracle of the kernel test). Sampling draws its Gumbel
    noise from a torch generator seeded with ``seed`` and the history index, so it is reproducible but does not
    reproduce the kernel's random stream."""
    B = logits.shape[0]
    scores = logits.float()
    words = st.params.cpu().numpy()
    eos = [int(e) for e in words[:8] if e >= 0]
    inv_temp = float(words[8:9].view(np.float32)[0])
    seed = int(words[10:12].view(np.uint64)[0]) % (2 ** 62)
    if inv_temp > 0:
        g = torch.Generator(device="cpu").manual_seed(int(seed) + int(st.count[0].item()))
        u = torch.rand(scores.shape, generator=g).clamp_(1e-7, 1 - 1e-7).to(scores.device)
        scores = scores * inv_temp - torch.log(-torch.log(u))
    width, bs, cap = st.table.shape[1], st.block_size, st.hist.shape[1]
    for b in range(B):
        c = int(st.count[b])
        st.count[b] = c + 1
        if int(st.finished[b]):
            if c < cap:
                st.hist[b, c] = -1
            continue
        row = torch.nan_to_num(scores[b], nan=float("-inf"))
        t = int((row == row.max()).nonzero()[0]) if row.numel() else 0
        p = int(st.pos[b]) + 1
        if c < cap:
            st.hist[b, c] = t
        if p + 1 >= int(st.limit[b]) or p // bs >= width or t in eos:
            st.finished[b] = 1
            st.slots[b] = -1
            continue
        st.tok[0, b], st.pos[b], st.lens[b] = t, p, p + 1
        blk = int(st.table[b, p // bs])
        st.slots[b] = -1 if blk < 0 else blk * bs + p % bs


def decode_advance(logits: torch.Tensor, st: DecodeState) -> None:
    """Pick the next token of every sequence from ``logits [B, >=V]`` and advance ``st`` in place, with the sampling
    settings of ``st.set_sampling``: temperature 0 is greedy, otherwise a sample from ``softmax(logits / temperature)``.
    Finished sequences (an end token chosen, the length ``st.limit`` reached) stop moving and record -1."""
    if not logits.is_cuda:
        return _advance_reference(logits, st)
    if logits.dtype != torch.float32 or logits.stride(-1) != 1:
        logits = logits.float().contiguous()
    B, width = st.table.shape
    rc = _lib.get_lib().mfb_decode_advance(
        logits.data_ptr(), int(logits.stride(0)), int(logits.shape[1]), int(B), st.tok.data_ptr(), st.pos.data_ptr(),
        st.lens.data_ptr(), st.slots.data_ptr(), st.table.data_ptr(), int(width), int(st.block_size), st.hist.data_ptr(),
        int(st.hist.shape[1]), st.count.data_ptr(), st.finished.data_ptr(), st.limit.data_ptr(), st.params.data_ptr(),
        _lib.stream_ptr())
    _lib.check(rc, "mfb_decode_advance")
    _lib.count_launch(1)


def fast_path_ok(gcfg, processors, streamer_batch: int, lockstep: bool) -> bool:
    """Whether a generation can run on the device loop: no history-dependent logits processors, no top-k / top-p
    warping, at most ``MAX_EOS`` end tokens, no lockstep stepping across expert-parallel replicas."""
    if lockstep or len(processors):
        return False
    if len(gcfg.eos_ids()) > MAX_EOS:
        return False
    if gcfg.do_sample:
        top_k, top_p = getattr(gcfg, "top_k", 0) or 0, getattr(gcfg, "top_p", 1.0)
        if top_k not in (0, None) or (top_p is not None and float(top_p) < 1.0):
            return False
        if not gcfg.temperature or float(gcfg.temperature) <= 0:
            return False
    return True


def read_burst(st: DecodeState, steps: int) -> List[List[int]]:
    """The tokens of the last ``steps`` replays, per sequence, up to (and including) the one that finished it. One
    device-to-host copy; resets the history for the next burst."""
    host = st.hist[:, :steps].cpu()            # synchronises with the replays
    st.count.zero_()
    out = []
    for row in host.tolist():
        toks = []
        for t in row:
            if t < 0:
                break
            toks.append(int(t))
        out.append(toks)
    return out
