"""Per-rank logging.

Counterpart of the reference's ``mindformers/tools/logger.py`` (``get_logger`` :456,
``LimitedRepeatHandler`` :149, stream redirection :254): every rank writes rotating
``output/log/rank_N/{info,error}.log`` files; only selected ranks print to the console; identical
messages can be rate-limited. Environment: ``LOG_MF_PATH`` (log directory), ``MF_LOG_SUFFIX``.
"""
from __future__ import annotations

import logging
import logging.handlers
import os
import sys
import time
from typing import Iterable, Optional

_FMT = "%(asctime)s - %(name)s[%(filename)s:%(lineno)d] - %(levelname)s - %(message)s"
_NAME = "mindformers_b200"


def _rank() -> int:
    return int(os.environ.get("RANK", os.environ.get("RANK_ID", "0")))


class LimitedRepeatFilter(logging.Filter):
    """Drop a message once it was emitted ``limit`` times within ``window`` seconds."""

    def __init__(self, limit: int = 0, window: float = 60.0):
        super().__init__()
        self.limit, self.window = limit, window
        self._seen: dict = {}

    def filter(self, record: logging.LogRecord) -> bool:
        if self.limit <= 0:
            return True
        key = (record.levelno, record.getMessage())
        now = time.time()
        count, first = self._seen.get(key, (0, now))
        if now - first > self.window:
            count, first = 0, now
        count += 1
        self._seen[key] = (count, first)
        return count <= self.limit


class StreamRedirector:
    """Context manager sending ``sys.stdout``/``sys.stderr`` writes to a logger."""

    def __init__(self, logger: logging.Logger, level: int = logging.INFO):
        self.logger, self.level = logger, level
        self._saved = None

    def write(self, text: str):
        text = text.rstrip()
        if text:
            self.logger.log(self.level, text)

    def flush(self):
        pass

    def __enter__(self):
        self._saved = (sys.stdout, sys.stderr)
        sys.stdout = sys.stderr = self
        return self

    def __exit__(self, *exc):
        sys.stdout, sys.stderr = self._saved
        return False


def get_logger(name: str = _NAME, *, to_std: Optional[bool] = None, stdout_ranks: Iterable[int] = (0,),
               log_dir: Optional[str] = None, file_level: int = logging.INFO, std_level: int = logging.INFO,
               max_bytes: int = 50 << 20, backup_count: int = 5, repeat_limit: int = 0,
               to_file: Optional[bool] = None) -> logging.Logger:
    """Return the framework logger, configuring handlers on first use."""
    log = logging.getLogger(name)
    if getattr(log, "_mf_configured", False):
        return log
    log.setLevel(logging.DEBUG)
    log.propagate = False
    rank = _rank()
    fmt = logging.Formatter(_FMT)
    show = (rank in set(stdout_ranks)) if to_std is None else to_std
    if show:
        sh = logging.StreamHandler(sys.stdout)
        sh.setLevel(std_level)
        sh.setFormatter(fmt)
        sh.addFilter(LimitedRepeatFilter(repeat_limit))
        log.addHandler(sh)
    if to_file is None:
        to_file = bool(os.environ.get("LOG_MF_PATH")) or log_dir is not None
    if to_file:
        base = log_dir or os.environ.get("LOG_MF_PATH") or os.path.join("output", "log")
        suffix = os.environ.get("MF_LOG_SUFFIX", "")
        rank_dir = os.path.join(base, f"rank_{rank}")
        os.makedirs(rank_dir, exist_ok=True)
        for fname, level in (("info", file_level), ("error", logging.ERROR)):
            path = os.path.join(rank_dir, f"{fname}{('_' + suffix) if suffix else ''}.log")
            fh = logging.handlers.RotatingFileHandler(path, maxBytes=max_bytes, backupCount=backup_count)
            fh.setLevel(level)
            fh.setFormatter(fmt)
            log.addHandler(fh)
    log._mf_configured = True
    return log


logger = get_logger()
