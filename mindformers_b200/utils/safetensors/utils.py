"""Directory probes (reference ``utils/safetensors/utils.py:23-74``)."""
from __future__ import annotations

import os

from ...checkpoint.io import is_hf_safetensors_dir  # noqa: F401  (same probe, one implementation)


def contains_safetensors_files(path: str) -> bool:
    return os.path.isdir(path) and any(f.endswith(".safetensors") for f in os.listdir(path))
