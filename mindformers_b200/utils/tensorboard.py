"""TensorBoard writer per rank (``mindformers/utils/tensorboard.py``: one writer, config dumped as text).

``torch.utils.tensorboard`` needs the ``tensorboard`` package; where it is absent the same scalars go to a
JSON-lines file (``scalars.jsonl``) with the same ``add_scalar`` / ``add_text`` interface, so monitors never
have to care which one they got.
"""
from __future__ import annotations

import json
import os
import time
from typing import Optional

_WRITER = None


class JsonlWriter:
    """Scalar writer used when neither ``tensorboardX`` nor ``torch.utils.tensorboard`` is importable: one JSON
    object per ``add_scalar`` / ``add_text`` call."""

    def __init__(self, log_dir: str):
        os.makedirs(log_dir, exist_ok=True)
        self.path = os.path.join(log_dir, "scalars.jsonl")
        self._f = open(self.path, "a")

    def add_scalar(self, tag, value, global_step=None, **kw):
        self._f.write(json.dumps({"tag": tag, "value": float(value), "step": global_step, "time": time.time()}) + "\n")

    def add_text(self, tag, text, global_step=None, **kw):
        self._f.write(json.dumps({"tag": tag, "text": str(text), "step": global_step}) + "\n")

    def flush(self):
        self._f.flush()

    def close(self):
        self._f.close()


def get_tensorboard_writer(log_dir: Optional[str] = None, queue_size: int = 10):
    global _WRITER
    if _WRITER is not None or log_dir is None:
        return _WRITER
    try:
        from torch.utils.tensorboard import SummaryWriter
        _WRITER = SummaryWriter(log_dir=log_dir, max_queue=queue_size)
    except Exception:
        _WRITER = JsonlWriter(log_dir)
    return _WRITER


def _flatten(prefix, obj, out):
    if isinstance(obj, dict):
        for k, v in obj.items():
            _flatten(f"{prefix}.{k}" if prefix else str(k), v, out)
    else:
        out[prefix] = obj


def write_args_to_tensorboard(config, writer=None):
    """Dumps every config leaf as a text entry named by its dotted path."""
    writer = writer or _WRITER
    if writer is None:
        return
    flat = {}
    _flatten("", config.to_dict() if hasattr(config, "to_dict") else dict(config), flat)
    for k, v in flat.items():
        writer.add_text(k, str(v), 0)


def close_tensorboard():
    global _WRITER
    if _WRITER is not None:
        _WRITER.close()
        _WRITER = None
