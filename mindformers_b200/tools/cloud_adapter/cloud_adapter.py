"""Mirroring run outputs to a remote location.

The reference syncs ``output/`` to ModelArts OBS through ``moxing`` (``mindformers/tools/cloud_adapter/cloud_adapter.py``:
``mox_adapter``, ``Local2ObsMonitor``, ``cloud_monitor``). Without a network the remote is any mounted path: the
same calls copy files there, with the retry loop and the keep-last policy of the reference.
"""
from __future__ import annotations

import functools
import os
import shutil
import time
from typing import Callable, Optional

from ..logger import logger


def mox_adapter(src_dir: str, target_dir: str, retry: int = 3, retry_time: float = 1.0, log: Callable = logger.info) -> bool:
    """Copy a file or a directory tree; retried ``retry`` times. Returns True on success."""
    for attempt in range(1, retry + 1):
        try:
            if os.path.isdir(src_dir):
                shutil.copytree(src_dir, target_dir, dirs_exist_ok=True)
            else:
                os.makedirs(os.path.dirname(target_dir) or ".", exist_ok=True)
                shutil.copy2(src_dir, target_dir)
            log(f"copied {src_dir} -> {target_dir}")
            return True
        except OSError as e:
            log(f"copy {src_dir} -> {target_dir} failed ({e}); attempt {attempt} of {retry}")
            time.sleep(retry_time)
    return False


class Local2ObsMonitor:
    """Callback: every ``upload_frequence`` steps (and at the end) mirror ``src_dir`` to ``target_dir/rank_<id>``;
    ``keep_last`` removes older checkpoint files from the remote copy."""

    def __init__(self, src_dir: str, target_dir: str, rank_id: Optional[int] = None, upload_frequence: int = 1,
                 keep_last: bool = True, retry: int = 3, retry_time: float = 1.0):
        self.src_dir = src_dir
        rank = int(os.environ.get("RANK", "0")) if rank_id is None else int(rank_id)
        self.target_dir = os.path.join(target_dir, f"rank_{rank}")
        self.freq, self.keep_last, self.retry, self.retry_time = max(1, upload_frequence), keep_last, retry, retry_time
        self.uploads = 0

    def _sync(self):
        if not os.path.isdir(self.src_dir):
            return
        if self.keep_last and os.path.isdir(self.target_dir):
            local = {os.path.relpath(os.path.join(r, f), self.src_dir) for r, _, fs in os.walk(self.src_dir) for f in fs}
            for r, _, fs in os.walk(self.target_dir):
                for f in fs:
                    rel = os.path.relpath(os.path.join(r, f), self.target_dir)
                    if rel not in local and f.endswith((".safetensors", ".ckpt", ".pt")):
                        os.remove(os.path.join(r, f))
        if mox_adapter(self.src_dir, self.target_dir, self.retry, self.retry_time):
            self.uploads += 1

    def on_step_end(self, ctx):
        if (ctx.cur_step_num if hasattr(ctx, "cur_step_num") else getattr(ctx, "step", 0)) % self.freq == 0:
            self._sync()

    def on_train_end(self, ctx):
        self._sync()


def cloud_monitor(target_dir: Optional[str] = None, src_dir: str = "./output"):
    """Decorator for a run function: mirror ``src_dir`` to ``target_dir`` (or ``$MFB200_REMOTE_SAVE_URL``) when it
    returns or raises."""

    def deco(fn):
        @functools.wraps(fn)
        def wrapper(*args, **kwargs):
            remote = target_dir or os.environ.get("MFB200_REMOTE_SAVE_URL")
            try:
                return fn(*args, **kwargs)
            finally:
                if remote:
                    mox_adapter(src_dir, remote)
        return wrapper
    return deco
