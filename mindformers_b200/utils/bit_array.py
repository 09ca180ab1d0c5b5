"""Fixed-size bit set used for CPU masks (reference ``mindformers/utils/bit_array.py``)."""
from __future__ import annotations

from typing import Iterable, List


class BitArray:
    """Fixed-size bit set over an integer (CPU masks for affinity): ``set``, ``clear``, ``test``, ranges to and from
    strings like ``0-3,8``."""

    def __init__(self, length: int = 0):
        if length < 0:
            raise ValueError("length must be non-negative")
        self.length = length
        self.bits = 0

    @classmethod
    def from_indices(cls, indices: Iterable[int], length: int = 0) -> "BitArray":
        idx = list(indices)
        out = cls(max(length, (max(idx) + 1) if idx else 0))
        for i in idx:
            out.set(i)
        return out

    def load_from_str(self, mask: str) -> "BitArray":
        """Comma-separated hexadecimal words, most significant first (the format of ``/proc/*/status``
        ``Cpus_allowed``)."""
        words = [w for w in mask.strip().split(",") if w]
        self.bits = int("".join(w.zfill(8) for w in words) or "0", 16)
        self.length = max(self.length, 32 * len(words))
        return self

    def set(self, i: int, value: bool = True):
        if i < 0:
            raise IndexError(i)
        self.length = max(self.length, i + 1)
        if value:
            self.bits |= 1 << i
        else:
            self.bits &= ~(1 << i)

    def get(self, i: int) -> bool:
        return bool((self.bits >> i) & 1)

    __getitem__ = get

    def get_marked_index(self) -> List[int]:
        return [i for i in range(self.length) if (self.bits >> i) & 1]

    def count(self) -> int:
        return bin(self.bits).count("1")

    def __and__(self, other: "BitArray") -> "BitArray":
        out = BitArray(max(self.length, other.length))
        out.bits = self.bits & other.bits
        return out

    def __or__(self, other: "BitArray") -> "BitArray":
        out = BitArray(max(self.length, other.length))
        out.bits = self.bits | other.bits
        return out

    def __sub__(self, other: "BitArray") -> "BitArray":
        out = BitArray(max(self.length, other.length))
        out.bits = self.bits & ~other.bits
        return out

    def to_mask_str(self) -> str:
        words = max(1, -(-self.length // 32))
        return ",".join(f"{(self.bits >> (32 * w)) & 0xFFFFFFFF:08x}" for w in reversed(range(words)))

    def __repr__(self):
        return f"BitArray({self.get_marked_index()})"
