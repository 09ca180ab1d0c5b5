"""Feature gates that depend on the software / hardware found at run time
(``mindformers/version_control.py``: version-dependent switches such as ``check_tft_valid:389``, ``is_910b:54``)."""
from __future__ import annotations

import functools
import os

import torch


@functools.lru_cache(None)
def device_capability():
    return torch.cuda.get_device_capability(0) if torch.cuda.is_available() else (0, 0)


def is_b200() -> bool:
    return device_capability()[0] == 10


def is_version_ge(current: str, base: str) -> bool:
    def parse(v):
        return [int("".join(c for c in p if c.isdigit()) or 0) for p in v.split("+")[0].split(".")[:3]]
    return parse(current) >= parse(base)


def check_symmetric_memory_valid() -> bool:
    """Peer-mapped buffers (fused TP / DP / MoE kernels) need torch's symmetric memory and more than one GPU."""
    try:
        import torch.distributed._symmetric_memory  # noqa: F401
    except Exception:
        return False
    return torch.cuda.is_available() and torch.cuda.device_count() > 1


def check_nvls_valid() -> bool:
    return check_symmetric_memory_valid() and os.environ.get("NCCL_NVLS_ENABLE", "1") != "0"


def check_tft_valid() -> bool:
    """Host-side fault tolerance (exception save, rollback on TREError) is switched on by ``MF_ENABLE_TFT``."""
    return bool(os.environ.get("MF_ENABLE_TFT") or os.environ.get("MS_ENABLE_TFT"))


def check_tre_valid() -> bool:
    flags = os.environ.get("MF_ENABLE_TFT", "") + os.environ.get("MS_ENABLE_TFT", "")
    return "TRE:1" in flags.replace(" ", "")


def check_delay_init_valid() -> bool:
    return is_version_ge(torch.__version__, "2.1.0")     # meta-device construction


def get_dropout(dropout_prob: float):
    return torch.nn.Dropout(p=dropout_prob)
