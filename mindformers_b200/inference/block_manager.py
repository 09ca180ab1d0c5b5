"""Host-side paged-KV bookkeeping: free-list block pool, per-sequence cache engines, block tables and slot maps.

Reference: ``modules/block_tables.py`` (``BlockTables.assemble_pa_full_inputs`` :65-96, ``assemble_pa_inc_inputs``
:98-121) and ``modules/cache_engine.py`` (``BlockMemPool`` :20-60, ``CacheEngine.prepare_cache`` :63-90). Running
out of blocks is a hard error (no preemption), as in the reference.
"""
from __future__ import annotations

from typing import List

import numpy as np


class BlockMemPool:
    """Free list of KV-cache block ids (reference ``modules/block_tables.py:20-60``)."""

    def __init__(self, num_blocks: int, block_size: int):
        self.num_blocks, self.block_size = num_blocks, block_size
        self.free: List[int] = list(range(num_blocks - 1, -1, -1))

    def allocate(self, n: int) -> List[int]:
        if n > len(self.free):
            raise RuntimeError(f"block pool is out of memory: {n} blocks requested, {len(self.free)} free")
        return [self.free.pop() for _ in range(n)]

    def release(self, blocks: List[int]):
        self.free.extend(reversed(blocks))

    @property
    def num_free(self) -> int:
        return len(self.free)


class CacheEngine:
    """Blocks owned by one sequence."""

    def __init__(self, pool: BlockMemPool):
        self.pool = pool
        self.blocks: List[int] = []
        self.num_tokens = 0

    def prepare_cache(self, num_new_tokens: int):
        total = self.num_tokens + num_new_tokens
        need = -(-total // self.pool.block_size) - len(self.blocks)
        if need > 0:
            self.blocks.extend(self.pool.allocate(need))
        self.num_tokens = total

    def reserve(self, total_tokens: int):
        """Own enough blocks for ``total_tokens`` cached tokens without caching any: the block table of a sequence
        then stays fixed while a device-side loop appends tokens."""
        need = -(-int(total_tokens) // self.pool.block_size) - len(self.blocks)
        if need > 0:
            self.blocks.extend(self.pool.allocate(need))

    def release(self):
        self.pool.release(self.blocks)
        self.blocks, self.num_tokens = [], 0

    def rollback(self, num_tokens: int):
        """Forget the last ``num_tokens`` cached tokens (rejected draft tokens); their slots are rewritten later."""
        self.num_tokens = max(0, self.num_tokens - int(num_tokens))


class BlockTables:
    """Block tables and slot mappings of a batch."""

    def __init__(self, num_blocks: int, block_size: int, seq_length: int):
        self.block_size = block_size
        self.max_blocks_per_seq = -(-seq_length // block_size)
        self.pool = BlockMemPool(num_blocks, block_size)
        self.engines: List[CacheEngine] = []

    def init_cache_engine(self, batch_size: int):
        self.clear_cache()
        self.engines = [CacheEngine(self.pool) for _ in range(batch_size)]

    def clear_cache(self):
        for e in self.engines:
            e.release()
        self.engines = []

    def _table(self) -> np.ndarray:
        t = np.full((len(self.engines), self.max_blocks_per_seq), -1, dtype=np.int32)
        for i, e in enumerate(self.engines):
            t[i, : len(e.blocks)] = e.blocks
        return t

    def assemble_pa_full_inputs(self, valid_lengths, active=None):
        """Prefill: allocate blocks for every prompt; returns (block_tables [B, max_blocks], slot_mapping [ΣL])."""
        slots = []
        for i, n in enumerate(valid_lengths):
            if active is not None and not active[i]:
                continue
            e = self.engines[i]
            start = e.num_tokens
            e.prepare_cache(int(n))
            pos = np.arange(start, start + int(n))
            blocks = np.asarray(e.blocks, dtype=np.int64)
            slots.append(blocks[pos // self.block_size] * self.block_size + pos % self.block_size)
        slot_mapping = np.concatenate(slots).astype(np.int32) if slots else np.zeros(0, np.int32)
        return self._table(), slot_mapping

    def assemble_pa_inc_inputs(self, active=None, num_new: int = 1):
        """Decode: one (or ``num_new``) more token per active sequence."""
        slots = []
        for i, e in enumerate(self.engines):
            if active is not None and not active[i]:
                slots.append(np.full(num_new, -1, dtype=np.int64))
                continue
            start = e.num_tokens
            e.prepare_cache(num_new)
            pos = np.arange(start, start + num_new)
            blocks = np.asarray(e.blocks, dtype=np.int64)
            slots.append(blocks[pos // self.block_size] * self.block_size + pos % self.block_size)
        return self._table(), np.concatenate(slots).astype(np.int32)

    def reserve(self, totals, active=None):
        """Reserve blocks for ``totals[i]`` tokens of every (active) sequence; returns the block tables."""
        for i, e in enumerate(self.engines):
            if active is None or active[i]:
                e.reserve(int(totals[i]))
        return self._table()

    def context_lens(self) -> np.ndarray:
        return np.asarray([e.num_tokens for e in self.engines], dtype=np.int32)
