"""Megatron ``.idx`` / ``.bin`` indexed datasets: reader (memory-mapped) and builder.

On-disk format (reference ``dataset/blended_datasets/indexed_dataset.py:34,122-200``): ``.idx`` =
``b"MMIDIDX\\x00\\x00"``, ``<Q`` version 1, ``<B`` dtype code, ``<Q`` sequence count, ``<Q`` document count,
int32 sequence lengths, int64 byte pointers, int64 document boundaries, optional int8 modes; ``.bin`` = raw tokens.
"""
from __future__ import annotations

import enum
import os
import struct
from typing import List, Optional, Sequence

import numpy as np

_MAGIC = b"MMIDIDX\x00\x00"
_DTYPES = {1: np.uint8, 2: np.int8, 3: np.int16, 4: np.int32, 5: np.int64, 6: np.float64, 7: np.float32, 8: np.uint16}
_CODES = {np.dtype(v): k for k, v in _DTYPES.items()}


class DType(enum.Enum):
    """Element-type codes of the ``.idx`` header (the Megatron on-disk format)."""
    uint8 = 1
    int8 = 2
    int16 = 3
    int32 = 4
    int64 = 5
    float64 = 6
    float32 = 7
    uint16 = 8

    @classmethod
    def code_from_dtype(cls, value) -> int:
        return cls[np.dtype(value).name].value

    @classmethod
    def dtype_from_code(cls, value: int):
        return getattr(np, cls(value).name)

    @staticmethod
    def size(key) -> int:
        """Bytes per element of a code or a dtype."""
        if isinstance(key, int):
            return np.dtype(DType.dtype_from_code(key)).itemsize
        return np.dtype(key).itemsize

    @staticmethod
    def optimal_dtype(cardinality: Optional[int]):
        """uint16 when every token id fits, else int32."""
        return np.uint16 if cardinality is not None and cardinality < 65500 else np.int32


def get_idx_path(prefix: str) -> str:
    return prefix + ".idx"


def get_bin_path(prefix: str) -> str:
    return prefix + ".bin"


def best_dtype(vocab_size: Optional[int]) -> type:
    return np.uint16 if vocab_size is not None and vocab_size < 65500 else np.int32


class IndexedDatasetBuilder:
    """Append token sequences, mark document ends, then ``finalize`` writes the index."""

    def __init__(self, bin_path: str, dtype=np.int32, multimodal: bool = False):
        self._bin = open(bin_path, "wb")
        self.dtype = np.dtype(dtype)
        self.multimodal = multimodal
        self.lengths: List[int] = []
        self.doc_indices: List[int] = [0]
        self.modes: List[int] = []

    def add_item(self, tokens: Sequence[int], mode: int = 0):
        arr = np.asarray(tokens, dtype=self.dtype)
        self._bin.write(arr.tobytes(order="C"))
        self.lengths.append(arr.size)
        if self.multimodal:
            self.modes.append(mode)

    def add_document(self, tokens: Sequence[int], lengths: Sequence[int], modes: Optional[Sequence[int]] = None):
        arr = np.asarray(tokens, dtype=self.dtype)
        self._bin.write(arr.tobytes(order="C"))
        self.lengths.extend(int(x) for x in lengths)
        self.doc_indices.append(len(self.lengths))
        if self.multimodal:
            self.modes.extend(modes if modes is not None else [0] * len(lengths))

    def end_document(self):
        self.doc_indices.append(len(self.lengths))

    def add_index(self, other_prefix: str):
        """Append another finished dataset of the same dtype."""
        other = IndexedDataset(other_prefix)
        if other.dtype != self.dtype:
            raise ValueError("cannot merge indexed datasets of different dtypes")
        offset = len(self.lengths)
        self.lengths.extend(other.sequence_lengths.tolist())
        self.doc_indices.extend((offset + other.document_indices[1:]).tolist())
        with open(get_bin_path(other_prefix), "rb") as f:
            while True:
                buf = f.read(1 << 24)
                if not buf:
                    break
                self._bin.write(buf)

    def finalize(self, idx_path: str):
        self._bin.close()
        lengths = np.asarray(self.lengths, dtype=np.int32)
        pointers = np.zeros(len(lengths), dtype=np.int64)
        if len(lengths) > 1:
            np.cumsum(lengths[:-1].astype(np.int64) * self.dtype.itemsize, out=pointers[1:])
        with open(idx_path, "wb") as f:
            f.write(_MAGIC)
            f.write(struct.pack("<Q", 1))
            f.write(struct.pack("<B", _CODES[self.dtype]))
            f.write(struct.pack("<Q", len(lengths)))
            f.write(struct.pack("<Q", len(self.doc_indices)))
            f.write(lengths.tobytes(order="C"))
            f.write(pointers.tobytes(order="C"))
            f.write(np.asarray(self.doc_indices, dtype=np.int64).tobytes(order="C"))
            if self.multimodal:
                f.write(np.asarray(self.modes, dtype=np.int8).tobytes(order="C"))


class _S3Bin:
    """Token data of an object-store ``.bin``: ranged reads of ``chunk`` bytes, the last chunk kept for the next
    request (sequential access, which is what the samplers mostly do, hits it)."""

    def __init__(self, path: str, chunk: int, client=None):
        self.path, self.chunk, self.client = path, max(1, int(chunk)), client
        self._start, self._data = 0, b""
        self.requests = 0

    def read(self, offset: int, nbytes: int) -> bytes:
        from . import utils_s3
        if not (self._start <= offset and offset + nbytes <= self._start + len(self._data)):
            self._start = offset
            self._data = utils_s3.read_range(self.path, offset, max(nbytes, self.chunk), self.client)
            self.requests += 1
        lo = offset - self._start
        return self._data[lo:lo + nbytes]


class IndexedDataset:
    """Random access to the sequences of a ``prefix.idx`` / ``prefix.bin`` pair."""

    def __init__(self, path_prefix: str, multimodal: bool = False, mmap: bool = True, object_storage_config=None,
                 s3_client=None):
        """``path_prefix`` may be an ``s3://bucket/key`` prefix: the index is downloaded once into
        ``object_storage_config.path_to_idx_cache`` and token data is fetched with ranged reads of
        ``bin_chunk_nbytes`` (``dataset/utils_s3.py``)."""
        self.path_prefix = path_prefix
        self.multimodal = multimodal
        self._s3 = None
        idx_file = get_idx_path(path_prefix)
        from . import utils_s3
        if utils_s3.is_s3_path(path_prefix):
            if object_storage_config is None:
                raise ValueError("an s3:// dataset prefix needs object_storage_config (S3Config)")
            idx_file = utils_s3.maybe_download_index(idx_file, object_storage_config, s3_client)
            self._s3 = _S3Bin(get_bin_path(path_prefix), object_storage_config.bin_chunk_nbytes, s3_client)
        with open(idx_file, "rb") as f:
            if f.read(9) != _MAGIC:
                raise ValueError(f"{idx_file} is not an indexed-dataset index")
            (version,) = struct.unpack("<Q", f.read(8))
            if version != 1:
                raise ValueError(f"unsupported index version {version}")
            (code,) = struct.unpack("<B", f.read(1))
            self.dtype = np.dtype(_DTYPES[code])
            (n_seq,) = struct.unpack("<Q", f.read(8))
            (n_doc,) = struct.unpack("<Q", f.read(8))
            offset = f.tell()
        idx = np.memmap(idx_file, mode="r", order="C")
        self.sequence_lengths = np.frombuffer(idx, dtype=np.int32, count=n_seq, offset=offset)
        offset += n_seq * 4
        self.sequence_pointers = np.frombuffer(idx, dtype=np.int64, count=n_seq, offset=offset)
        offset += n_seq * 8
        self.document_indices = np.frombuffer(idx, dtype=np.int64, count=n_doc, offset=offset)
        offset += n_doc * 8
        self.sequence_modes = np.frombuffer(idx, dtype=np.int8, count=n_seq, offset=offset) if multimodal else None
        self._idx_map = idx
        if self._s3 is not None:
            self._bin = None
        elif mmap:
            self._bin = np.memmap(get_bin_path(path_prefix), mode="r", order="C")
        else:
            self._bin = np.fromfile(get_bin_path(path_prefix), dtype=np.uint8)

    def __len__(self):
        return len(self.sequence_lengths)

    def get(self, idx: int, offset: int = 0, length: Optional[int] = None) -> np.ndarray:
        n = int(self.sequence_lengths[idx]) - offset
        if length is not None:
            n = min(n, length)
        start = int(self.sequence_pointers[idx]) + offset * self.dtype.itemsize
        if self._s3 is not None:
            return np.frombuffer(self._s3.read(start, n * self.dtype.itemsize), dtype=self.dtype, count=n)
        return np.frombuffer(self._bin, dtype=self.dtype, count=n, offset=start)

    def __getitem__(self, idx):
        if isinstance(idx, slice):
            return [self.get(i) for i in range(*idx.indices(len(self)))]
        return self.get(int(idx))

    @staticmethod
    def exists(path_prefix: str) -> bool:
        return os.path.exists(get_idx_path(path_prefix)) and os.path.exists(get_bin_path(path_prefix))
