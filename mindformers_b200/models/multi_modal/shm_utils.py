"""Passing image / audio features from a serving front end to the model workers through POSIX shared memory.

A front end that owns the pre-processing cannot put a float array into a stream of token ids, so it parks the array in
a shared-memory segment and sends two NEGATIVE int64 "tokens" in its place: one names the segment, one gives the
array's shape. The worker recognises them by their sign, decodes both, maps the segment and gets the array back.
Reference: ``models/multi_modal/shm_utils.py`` (``create_shm`` :32, ``release_shared_memory`` :49,
``encode_shm_name_to_int64`` :64, ``encode_shape_to_int64`` :106, the two decoders :149 / :186, ``get_data_from_shm`` :232).

Encodings used here (both leave the sign bit free, the value is negated at the end):

* name: Python names its segments ``<prefix><hex digits>``; the prefix is dropped, and the value is
  ``[4 bits: number of hex digits (<= 12)] [48 bits: the digits] [8 bits: checksum]``;
* shape: ``[3 bits: rank (1..6)] [rank fields of 56 // rank bits] [4 bits: checksum]``.

The checksums catch an id that merely happens to be negative.
"""
from __future__ import annotations

import os
from multiprocessing import shared_memory
from typing import Sequence, Tuple

import numpy as np

try:
    from multiprocessing.shared_memory import _SHM_NAME_PREFIX as _RAW_PREFIX
except ImportError:          # pragma: no cover - other platforms
    _RAW_PREFIX = "/psm_"
SHM_NAME_PREFIX = _RAW_PREFIX.lstrip("/")        # ``SharedMemory.name`` reports the name without the leading slash
MAX_SHM_SIZE = int(os.environ.get("MAX_SHM_SIZE", 10 ** 9))
_MAX_DIGITS = 12


def _checksum8(value: int) -> int:
    s = 0
    while value:
        s = (s * 31 + (value & 0xFF)) & 0xFF
        value >>= 8
    return s ^ 0x5A


def create_shm(size: int, shm_name_save_path: str):
    """A new segment of ``size`` bytes; its name is appended to ``shm_name_save_path`` so that a clean-up pass can
    unlink what a crashed process left behind."""
    if not isinstance(size, int) or size <= 0:
        raise ValueError("Size must be a positive integer.")
    if size > MAX_SHM_SIZE:
        raise ValueError(f"Size exceeds the maximum allowed limit of {MAX_SHM_SIZE} bytes.")
    shm = shared_memory.SharedMemory(create=True, size=size)
    fd = os.open(shm_name_save_path, os.O_WRONLY | os.O_CREAT | os.O_APPEND, 0o600)
    with os.fdopen(fd, "a", encoding="utf-8") as f:
        f.write(shm.name + "\n")
    return shm


def release_shared_memory(file_path: str) -> int:
    """Unlink every segment named in ``file_path`` (segments that are gone already are skipped); returns the count."""
    if not os.path.exists(file_path):
        raise FileNotFoundError(f"{file_path} does not exist")
    n = 0
    with open(file_path, "r", encoding="utf-8") as f:
        names = [line.strip() for line in f if line.strip()]
    for name in names:
        try:
            shm = shared_memory.SharedMemory(name=name)
        except FileNotFoundError:
            continue
        shm.close()
        shm.unlink()
        n += 1
    return n


def encode_shm_name_to_int64(name: str) -> int:
    name = name.lstrip("/")
    digits = name[len(SHM_NAME_PREFIX):] if name.startswith(SHM_NAME_PREFIX) else name
    if not digits or len(digits) > _MAX_DIGITS:
        raise ValueError(f"shared-memory name {name!r}: 1 to {_MAX_DIGITS} hexadecimal digits after the prefix are supported")
    try:
        payload = int(digits, 16)
    except ValueError as e:
        raise ValueError(f"shared-memory name {name!r} is not hexadecimal after its prefix") from e
    body = (len(digits) << 48) | payload
    return -((body << 8) | _checksum8(body))


def decode_shm_name_from_int64(encoded_value: int) -> str:
    v = -int(encoded_value)
    if v <= 0:
        raise ValueError("not an encoded shared-memory name")
    body, check = v >> 8, v & 0xFF
    if _checksum8(body) != check:
        raise ValueError("checksum mismatch: the value is not an encoded shared-memory name")
    n = body >> 48
    if not 1 <= n <= _MAX_DIGITS:
        raise ValueError("invalid name length")
    return SHM_NAME_PREFIX + format(body & ((1 << 48) - 1), f"0{n}x")


def encode_shape_to_int64(shape: Sequence[int]) -> int:
    rank = len(shape)
    if not 1 <= rank <= 6:
        raise ValueError("Shape must have 1 to 6 dimensions")
    bits = 56 // rank
    packed = 0
    for d in shape:
        d = int(d)
        if d < 0 or d >= (1 << bits):
            raise ValueError(f"Dimension {d} is too large, max allowed is {(1 << bits) - 1} at rank {rank}")
        packed = (packed << bits) | d
    body = (rank << 56) | packed                 # the rank sits at a fixed position above the 56 dimension bits
    return -((body << 4) | (_checksum8(body) & 0xF))


def decode_shape_from_int64(encoded_value: int) -> Tuple[int, ...]:
    v = -int(encoded_value)
    if v <= 0:
        raise ValueError("not an encoded shape")
    body, check = v >> 4, v & 0xF
    if (_checksum8(body) & 0xF) != check:
        raise ValueError("checksum mismatch: the value is not an encoded shape")
    rank = body >> 56
    if not 1 <= rank <= 6:
        raise ValueError("invalid rank")
    bits = 56 // rank
    return tuple((body >> (bits * (rank - 1 - i))) & ((1 << bits) - 1) for i in range(rank))


def put_data_to_shm(array: np.ndarray, shm_name_save_path: str) -> Tuple[int, int]:
    """Front-end side: copy ``array`` into a new segment; returns ``(encoded name, encoded shape)``."""
    arr = np.ascontiguousarray(array)
    shm = create_shm(int(arr.nbytes), shm_name_save_path)
    np.ndarray(arr.shape, dtype=arr.dtype, buffer=shm.buf)[...] = arr
    name = shm.name
    shm.close()
    return encode_shm_name_to_int64(name), encode_shape_to_int64(arr.shape)


def get_data_from_shm(shm_name_value: int, shape_value: int, dtype=np.float32, unlink: bool = True) -> np.ndarray:
    """Worker side: the array behind the two encoded values (copied out; the segment is unlinked unless ``unlink=False``)."""
    name = decode_shm_name_from_int64(shm_name_value)
    shape = decode_shape_from_int64(shape_value)
    shm = shared_memory.SharedMemory(name=name)
    try:
        out = np.ndarray(shape, dtype=dtype, buffer=shm.buf).copy()
    finally:
        shm.close()
        if unlink:
            try:
                shm.unlink()
            except FileNotFoundError:
                pass
    return out
