"""ctypes binding of the in-tree sm_100a kernel library (``lib/libmfb200.so``).

The library exposes plain ``extern "C"`` entry points that take raw device pointers and a CUDA
stream, so it needs no torch headers and builds in seconds. On a machine with a GPU the library
must be present: a missing or stale ``.so`` raises instead of silently falling back to PyTorch.
"""
from __future__ import annotations

import ctypes
import os
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
KERNEL_LIB_PATH = os.path.join(_HERE, "lib", "libmfb200.so")
DATA_LIB_PATH = os.path.join(_HERE, "lib", "libmfb200_data.so")
ABI_VERSION = 2

_lock = threading.Lock()
_lib = None
_launch_count = 0  # kernels launched through this binding (read by the benchmark)

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_ll = ctypes.c_longlong
c_float = ctypes.c_float


class KernelLibraryError(RuntimeError):
    """The sm_100a kernel library is missing, stale, or one of its entry points returned an error code."""

    pass


def _declare(lib):
    def sig(name, args):
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = c_int
        return fn

    P, I, L, F = c_void_p, c_int, c_ll, c_float
    lib.mfb_last_error.restype = ctypes.c_char_p
    lib.mfb_abi_version.restype = c_int
    sig("mfb_gemm_bf16", [P, P, P, I, I, I, I, I, I, I, I, I, I, I, P, P, P, I, P, I, P])
    sig("mfb_gemm_bf16_decode_supported", [I, I, I])
    sig("mfb_gemm_bf16_decode", [P, P, P, P, I, I, I, L, L, L, I, P, P])
    sig("mfb_gemm_bf16_pair", [P, P, P, I, I, I, I, I, I, I, I, I, P, I, P, I, P])
    lib.mfb_gemm_pair_workspace_bytes.argtypes = []
    lib.mfb_gemm_pair_workspace_bytes.restype = L
    sig("mfb_gemm_pair_plan", [I, I, I, I, I, P, P])
    sig("mfb_rmsnorm_fwd", [P, P, P, P, P, P, I, I, F, P])
    sig("mfb_rmsnorm_bwd_parts", [I])
    sig("mfb_rmsnorm_bwd", [P, P, P, P, P, P, P, P, I, P, I, I, P])
    sig("mfb_headnorm_fwd", [P, P, P, I, I, I, L, F, P])
    sig("mfb_swiglu_fwd", [P, P, L, I, P])
    sig("mfb_swiglu_bwd", [P, P, P, L, I, P])
    sig("mfb_rope", [P, P, P, P, L, I, I, I, L, I, I, I, P])
    sig("mfb_embedding_fwd", [P, P, P, L, I, I, I, P])
    sig("mfb_embedding_bwd", [P, P, P, L, I, I, I, P])
    sig("mfb_accum_bf16_to_f32", [P, P, L, F, I, P])
    sig("mfb_add_bf16", [P, P, P, L, P])
    sig("mfb_ce_stats", [P, I, P, P, P, P, L, I, L, I, P])
    sig("mfb_ce_bwd", [P, P, I, P, P, P, L, I, L, I, P])
    sig("mfb_grad_sumsq_scratch", [])
    sig("mfb_grad_sumsq", [P, I, L, P, P, I, P])
    sig("mfb_adamw", [P, P, P, P, P, I, P, P, L, L, F, F, F, F, F, F, F, F, F, F, P])
    sig("mfb_split_master", [P, P, P, L, P])
    sig("mfb_join_master", [P, P, P, L, P])
    sig("mfb_flash_attn_fwd", [P, P, P, P, P, I, I, I, I, I, L, L, L, L, I, F, P, P])
    sig("mfb_flash_attn_fwd2_varlen", [P, P, P, P, P, P, I, I, I, I, I, L, L, L, L, I, I, F, P, P])
    sig("mfb_flash_attn_bwd2_varlen", [P] * 12 + [I, I, I, I, I] + [L] * 8 + [I, I, F, P, P])
    lib.mfb_tp_set_rs_interleave.argtypes = [I]
    lib.mfb_tp_set_rs_interleave.restype = None
    lib.mfb_tp_set_pair.argtypes = [I]
    lib.mfb_tp_set_pair.restype = None
    lib.mfb_flash_attn_set_bwd_variant.argtypes = [I]
    lib.mfb_flash_attn_set_bwd_variant.restype = None
    lib.mfb_flash_attn_bwd2_set_split.argtypes = [I]
    lib.mfb_flash_attn_bwd2_set_split.restype = None
    lib.mfb_flash_attn_bwd_scratch_bytes_ex.argtypes = [I, I, I, I, I]
    lib.mfb_flash_attn_bwd_scratch_bytes_ex.restype = L
    lib.mfb_flash_attn_set_fwd_variant.argtypes = [I]
    lib.mfb_flash_attn_set_fwd_variant.restype = None
    lib.mfb_flash_attn_fwd2_set_poly.argtypes = [I]
    lib.mfb_flash_attn_fwd2_set_poly.restype = None
    sig("mfb_flash_attn_fwd_mla", [P, P, P, P, P, I, I, I, I, I, L, L, L, L, I, I, F, P, P])
    lib.mfb_flash_attn_bwd_scratch_bytes.argtypes = [I, I, I]
    lib.mfb_flash_attn_bwd_scratch_bytes.restype = L
    sig("mfb_flash_attn_bwd", [P] * 10 + [I, I, I, I] + [L] * 8 + [I, F, P, P])
    sig("mfb_reshape_and_cache", [P, P, P, P, P, L, I, L, L, P])
    sig("mfb_paged_decode_attention", [P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, P])
    sig("mfb_paged_decode_splits", [I, I, I, I])
    lib.mfb_paged_decode_scratch_bytes.argtypes = [I, I, I, I]
    lib.mfb_paged_decode_scratch_bytes.restype = L
    sig("mfb_gemm_fp8_decode", [P, P, P, P, L, P, I, I, I, L, L, L, I, I, P, P, P, P, P, P])
    sig("mfb_gemm_fp8_decode_supported", [I, I, I, I])
    lib.mfb_gemm_fp8_enable_ksplit.argtypes = [I]
    lib.mfb_gemm_fp8_enable_ksplit.restype = None
    sig("mfb_gemm_fp8_ksplit", [I, I, I, I, L])
    sig("mfb_mla_decode_attention", [P, P, P, P, P, P, I, I, I, I, I, I, F, P, P])
    sig("mfb_mla_decode_splits", [I, I, I])
    lib.mfb_mla_decode_set_variant.argtypes = [I]
    lib.mfb_mla_decode_set_variant.restype = None
    sig("mfb_mla_decode_get_variant", [])
    lib.mfb_mla_decode_scratch_bytes.argtypes = [I, I, I]
    lib.mfb_mla_decode_scratch_bytes.restype = L
    sig("mfb_gather_cache", [P, P, P, P, I, I, I, I, I, P])
    lib.mfb_ll_allreduce_buffer_bytes.argtypes = [I, L]
    lib.mfb_ll_allreduce_buffer_bytes.restype = L
    sig("mfb_ll_allreduce_state_words", [])
    sig("mfb_ll_allreduce_init", [P, L, P])
    sig("mfb_ll_allreduce", [P, P, L, L, I, I, P, P, P, P])
    sig("mfb_dp_reduce_scratch", [])
    sig("mfb_dp_flag_words", [])
    sig("mfb_dp_reduce", [I, I, I, L, L, P, P, P, P, P, I, P, P])
    sig("mfb_dp_bucket_rows", [])
    sig("mfb_dp_adamw_publish", [I, I, I, I, L, L, L, P, P, P, P, P, P, P, P, L, F, F, F, F, F, F, F, F, F, F, P, P])
    sig("mfb_dp_wait_published", [I, I, I, I, P, P, P])
    sig("mfb_dp_announce", [I, I, I, I, P, P])
    sig("mfb_dp_reduce_bucket", [I, I, I, I, L, L, P, P, P, P, P, I, P, P])
    sig("mfb_dp_adamw_allgather", [I, I, I, L, L, P, P, P, P, P, P, P, P, L, F, F, F, F, F, F, F, F, F, F, P, P])
    sig("mfb_router_fwd", [P, P, P, P, P, P, I, I, I, I, I, I, I, F, P])
    sig("mfb_router_bwd", [P, P, P, P, P, I, I, I, I, I, F, P])
    sig("mfb_moe_flag_words", [])
    sig("mfb_moe_rank", [P, I, I, P, P, P])
    sig("mfb_moe_plan", [I, I, P, I, I, I] + [P] * 11)
    sig("mfb_moe_scatter", [I] * 7 + [P] * 12)
    sig("mfb_moe_barrier", [I, I, P, I, P, P, P])
    sig("mfb_moe_gather", [I] * 7 + [P] * 9)
    sig("mfb_flash_attn_fwd_ex", [P, P, P, P, P, I, I, I, I, I, L, L, L, L, I, I, F, P, P])
    sig("mfb_flash_attn_bwd_ex", [P] * 10 + [I, I, I, I, I] + [L] * 8 + [I, I, F, P, P])
    sig("mfb_cp_flag_words", [])
    sig("mfb_cp_gather", [I, I, I, I, I, L, I, P, P, P, P, P])
    sig("mfb_cp_reduce_scatter", [I, I, I, I, I, L, I, P, P, P, P, P])
    sig("mfb_cp_barrier", [I, I, I, I, P, P, P])
    sig("mfb_gemm_fp8_blockscaled", [P, P, P, P, L, P, I, I, I, L, L, L, I, I, P, P, P, P])
    sig("mfb_quant_act_1x128", [P, L, P, L, P, L, L, I, P])
    if hasattr(lib, "mfb_gemm_pair_set_band"):
        lib.mfb_gemm_pair_set_band.argtypes = [I]
        lib.mfb_gemm_pair_set_band.restype = None
    if hasattr(lib, "mfb_flash_attn_bwd2_set_probe"):
        lib.mfb_flash_attn_bwd2_set_probe.argtypes = [I]
        lib.mfb_flash_attn_bwd2_set_probe.restype = None
    sig("mfb_reshape_and_cache_int8", [P, P, P, P, P, P, P, L, I, I, L, L, P])
    sig("mfb_gather_cache_int8", [P, P, P, P, P, I, I, I, I, I, I, P])
    sig("mfb_decode_advance", [P, I, I, I, P, P, P, P, P, I, I, P, I, P, P, P, P, P])
    sig("mfb_paged_decode_tc_supported", [I, I, I, I])
    sig("mfb_paged_decode_tc_splits", [I, I, I])
    sig("mfb_paged_decode_attention_tc", [P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, P, P])
    sig("mfb_paged_decode_attention_ex", [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, P])
    sig("mfb_gemm_w8a8", [P, P, P, P, P, P, I, I, I, L, L, L, P, P])
    sig("mfb_quant_act_int8", [P, L, P, L, P, P, L, I, P])
    # optional entry points (present once their source file is part of the build)
    for name, args in _OPTIONAL.items():
        if hasattr(lib, name):
            sig(name, args)


_OPTIONAL: dict = {}


def optional_entry(name, args):
    """Register the signature of an entry point that later source files add to the library."""
    _OPTIONAL[name] = args
    if _lib is not None and hasattr(_lib, name):
        fn = getattr(_lib, name)
        fn.argtypes = args
        fn.restype = c_int


def available() -> bool:
    return os.path.exists(KERNEL_LIB_PATH)


def get_lib():
    """Load (once) and return the kernel library."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(KERNEL_LIB_PATH):
            raise KernelLibraryError(
                f"{KERNEL_LIB_PATH} is missing: run `python -m mindformers_b200.ops.build` "
                "(the CUDA path never falls back to PyTorch on a GPU)")
        lib = ctypes.CDLL(KERNEL_LIB_PATH)
        got = lib.mfb_abi_version()
        if got != ABI_VERSION:
            raise KernelLibraryError(f"kernel library ABI {got} != expected {ABI_VERSION}; rebuild it")
        _declare(lib)
        # kernel variants that can be switched for A/B measurements
        if os.environ.get("MFB_FP8_KSPLIT", "1") == "0":
            lib.mfb_gemm_fp8_enable_ksplit(0)
        if os.environ.get("MFB_FA_BWD", "2") == "1":
            lib.mfb_flash_attn_set_bwd_variant(1)
        if os.environ.get("MFB_FA_FWD", "2") == "1":
            lib.mfb_flash_attn_set_fwd_variant(1)
        if os.environ.get("MFB_FA_POLY"):
            lib.mfb_flash_attn_fwd2_set_poly(int(os.environ["MFB_FA_POLY"]))
        if os.environ.get("MFB_MLA_DECODE", "single") == "cluster":
            lib.mfb_mla_decode_set_variant(1)
        _lib = lib
    return _lib


def check(rc: int, what: str):
    if rc != 0:
        msg = get_lib().mfb_last_error().decode(errors="replace")
        raise KernelLibraryError(f"{what} failed (code {rc}): {msg}")


def stream_ptr() -> int:
    """Raw handle of the current CUDA stream of the current device (the direct binding: building a
    ``torch.cuda.Stream`` object per kernel launch costs more host time than the launch itself)."""
    return _raw_stream(torch.cuda.current_device())


try:
    _raw_stream = torch._C._cuda_getCurrentRawStream
except AttributeError:          # CPU-only builds of torch
    def _raw_stream(device_index: int) -> int:
        return torch.cuda.current_stream(device_index).cuda_stream


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def count_launch(n: int = 1):
    global _launch_count
    _launch_count += n


def launch_count() -> int:
    return _launch_count


def reset_launch_count():
    global _launch_count
    _launch_count = 0


_status_words: dict = {}


def status_word(device) -> torch.Tensor:
    """Per-device pair of int32 words that kernels report through. Word 0 takes the code of the first bounded wait
    that ran out (kernels get its address); word 1, right behind it, is set by the expert-parallel plan kernel when
    a receive buffer overflowed, so that an earlier time-out code cannot hide an overflow or the other way round."""
    key = torch.device(device).index or 0
    t = _status_words.get(key)
    if t is None:
        t = torch.zeros(2, dtype=torch.int32, device=device)
        _status_words[key] = t
    return t


def read_status(device=None) -> int:
    """Synchronising read of the wait status (0 = every bounded wait completed)."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    return int(status_word(device)[0].item())


def read_status_words(device=None):
    """Synchronising read of ``(wait status, expert-parallel overflow flag)``."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    a, b = status_word(device).tolist()
    return int(a), int(b)


class DeviceWaitTimeout(RuntimeError):
    """A bounded device-side wait (mbarrier phase, peer flag) ran out: the step's results are incomplete."""


_STATUS_NAMES = {1: "TMA producer wait", 2: "MMA issuer wait", 3: "epilogue wait", 4: "peer flag wait (another rank "
                 "did not arrive)", 5: "bad kernel argument"}


def raise_on_status(code: int, where: str = ""):
    if code:
        raise DeviceWaitTimeout(f"device status {code} ({_STATUS_NAMES.get(code, 'unknown')}) {where}: a bounded wait "
                                "inside a kernel ran out, so its output is incomplete; the run cannot continue on it")
