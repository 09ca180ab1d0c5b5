"""numpy front-end of the native index builders (``ops/csrc/data_helpers.cpp``).

The shared library is built in-tree by ``mindformers_b200.ops.build``; if it is missing it is compiled on first
use (g++ only, about a second), as the reference does with ``make`` (``dataset/blended_datasets/utils.py:22-33``).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

from ..ops import _lib as _k

_LIB = None


def compile_helpers():
    """Build ``libmfb200_data.so`` from source (CPU only)."""
    here = os.path.dirname(os.path.abspath(_k.__file__))
    src = os.path.join(here, "csrc", "data_helpers.cpp")
    os.makedirs(os.path.dirname(_k.DATA_LIB_PATH), exist_ok=True)
    tmp = _k.DATA_LIB_PATH + f".{os.getpid()}.tmp"
    subprocess.run(["g++", "-O3", "-std=c++17", "-fPIC", "-shared", src, "-o", tmp], check=True)
    os.replace(tmp, _k.DATA_LIB_PATH)


def _lib():
    global _LIB
    if _LIB is None:
        if not os.path.exists(_k.DATA_LIB_PATH):
            compile_helpers()
        lib = ctypes.CDLL(_k.DATA_LIB_PATH)
        P, I32, I64, D = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_double
        lib.mfb_num_samples.argtypes = [I64, I64, I32, I32, I32]
        lib.mfb_num_samples.restype = I64
        lib.mfb_build_sample_idx.argtypes = [P, P, I64, I32, I64, I64, I32, I32, P]
        lib.mfb_build_sample_idx.restype = ctypes.c_int
        lib.mfb_build_blending_indices.argtypes = [P, P, P, I32, I64]
        lib.mfb_build_exhaustive_blending_indices.argtypes = [P, P, P, I32]
        lib.mfb_build_mapping.argtypes = [P, I64, P, I32, ctypes.c_uint64, I32, D, I32, I32, P]
        lib.mfb_build_mapping.restype = I64
        lib.mfb_build_blocks_mapping.argtypes = [P, I64, P, P, I32, ctypes.c_uint64, I32, I32, I32, P]
        lib.mfb_build_blocks_mapping.restype = I64
        _LIB = lib
    return _LIB


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def build_sample_idx(sizes, doc_idx, seq_length: int, num_epochs: int, tokens_per_epoch: int,
                     drop_last_partial_sequence: bool = True, add_extra_token_to_sequence: int = 1) -> np.ndarray:
    sizes = np.ascontiguousarray(sizes, dtype=np.int32)
    doc_idx = np.ascontiguousarray(doc_idx, dtype=np.int32)
    lib = _lib()
    n = lib.mfb_num_samples(num_epochs, tokens_per_epoch, seq_length, int(drop_last_partial_sequence),
                            add_extra_token_to_sequence)
    out = np.zeros((n + 1, 2), dtype=np.int64)
    rc = lib.mfb_build_sample_idx(_ptr(sizes), _ptr(doc_idx), doc_idx.shape[0], seq_length, num_epochs,
                                  tokens_per_epoch, int(drop_last_partial_sequence), add_extra_token_to_sequence,
                                  _ptr(out))
    if rc:
        raise ValueError("build_sample_idx: invalid arguments")
    return out


def build_blending_indices(dataset_index: np.ndarray, dataset_sample_index: np.ndarray, weights, num_datasets: int,
                           size: int, verbose: bool = False):
    w = np.ascontiguousarray(weights, dtype=np.float64)
    assert dataset_index.dtype == np.int16 and dataset_sample_index.dtype == np.int64
    _lib().mfb_build_blending_indices(_ptr(dataset_index), _ptr(dataset_sample_index), _ptr(w), num_datasets, size)
    if verbose:
        for d in range(num_datasets):
            print(f"   dataset {d}, input: {w[d]:.4f}, achieved: {(dataset_index[:size] == d).mean():.4f}")


def build_exhaustive_blending_indices(dataset_index: np.ndarray, dataset_sample_index: np.ndarray, sizes,
                                      num_datasets: int):
    s = np.ascontiguousarray(sizes, dtype=np.int64)
    _lib().mfb_build_exhaustive_blending_indices(_ptr(dataset_index), _ptr(dataset_sample_index), _ptr(s), num_datasets)


def build_mapping(docs, sizes, num_epochs: int, max_num_samples: int, max_seq_length: int, short_seq_prob: float,
                  seed: int, verbose: bool = False, min_num_sent: int = 2) -> np.ndarray:
    docs = np.ascontiguousarray(docs, dtype=np.int64)
    sizes = np.ascontiguousarray(sizes, dtype=np.int32)
    lib = _lib()
    args = (_ptr(docs), docs.shape[0] - 1, _ptr(sizes), num_epochs, max_num_samples, max_seq_length,
            float(short_seq_prob), seed, min_num_sent)
    n = lib.mfb_build_mapping(*args, None)
    if n < 0:
        raise ValueError("build_mapping: invalid arguments")
    out = np.zeros((n, 3), dtype=np.int64)
    lib.mfb_build_mapping(*args, _ptr(out))
    return out


def build_blocks_mapping(docs, sizes, titles_sizes, num_epochs: int, max_num_samples: int, max_seq_length: int,
                         seed: int, verbose: bool = False, use_one_sent_blocks: bool = False) -> np.ndarray:
    docs = np.ascontiguousarray(docs, dtype=np.int64)
    sizes = np.ascontiguousarray(sizes, dtype=np.int32)
    titles = np.ascontiguousarray(titles_sizes, dtype=np.int32)
    lib = _lib()
    args = (_ptr(docs), docs.shape[0] - 1, _ptr(sizes), _ptr(titles), num_epochs, max_num_samples, max_seq_length,
            seed, int(use_one_sent_blocks))
    n = lib.mfb_build_blocks_mapping(*args, None)
    if n < 0:
        raise ValueError("build_blocks_mapping: invalid arguments")
    out = np.zeros((n, 4), dtype=np.int64)
    lib.mfb_build_blocks_mapping(*args, _ptr(out))
    return out
