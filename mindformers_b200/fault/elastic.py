"""Restart-from-checkpoint supervision (the ARF / TRE roles of the reference's fault-tolerance runtime, host side).

``run_with_restarts(train_fn, ...)`` runs ``train_fn(attempt, resume_dir)`` and, when it raises a recoverable error
(``RankFailure``, a ``RuntimeError`` whose message starts with ``TREError``, a collective timeout), tears the process
group down, waits for the surviving ranks at a store barrier and calls it again with ``resume_training`` pointing at the
newest checkpoint that every rank has (``checkpoint/resume.py``). ``ElasticRunner`` is the same loop as an object for
launchers that own the store. The GPU is never asked to time out: detection happens on the host (heartbeats, process-group
timeouts), and a rank only leaves between steps.
"""
from __future__ import annotations

import time
from typing import Callable, Optional

import torch.distributed as dist

from ..tools.logger import get_logger
from .heartbeat import RankFailure

logger = get_logger()

RECOVERABLE_PREFIXES = ("TREError", "NCCL", "ProcessGroup", "Timed out", "timeout")


def is_recoverable(exc: BaseException) -> bool:
    if isinstance(exc, RankFailure):
        return True
    if isinstance(exc, (RuntimeError, dist.DistBackendError if hasattr(dist, "DistBackendError") else RuntimeError)):
        msg = str(exc)
        return any(p in msg for p in RECOVERABLE_PREFIXES)
    return False


def run_with_restarts(train_fn: Callable[[int, Optional[str]], object], checkpoint_dir: Optional[str] = None,
                      max_restarts: int = 3, backoff_s: float = 1.0, on_restart: Optional[Callable[[int, BaseException], None]] = None):
    attempt = 0
    while True:
        try:
            return train_fn(attempt, checkpoint_dir if attempt > 0 else None)
        except BaseException as exc:  # noqa: BLE001
            if not is_recoverable(exc) or attempt >= max_restarts:
                raise
            attempt += 1
            logger.warning("attempt %d failed with %s: %s; restarting from the last common checkpoint", attempt, type(exc).__name__, exc)
            if dist.is_available() and dist.is_initialized():
                try:
                    dist.destroy_process_group()
                except Exception:  # noqa: BLE001
                    pass
            if on_restart is not None:
                on_restart(attempt, exc)
            time.sleep(backoff_s * attempt)


class ElasticRunner:
    """Supervises a training function: restarts it from the latest consistent checkpoint after a failure, up to
    ``max_restarts`` times (the host-side part of the reference's fault-tolerant training,
    ``core/callback/callback.py`` ``TrainFaultTolerance``)."""

    def __init__(self, checkpoint_dir: str, max_restarts: int = 3, backoff_s: float = 1.0):
        self.checkpoint_dir, self.max_restarts, self.backoff_s = checkpoint_dir, max_restarts, backoff_s
        self.restarts = 0

    def run(self, train_fn):
        def hook(attempt, exc):
            self.restarts = attempt
        return run_with_restarts(train_fn, self.checkpoint_dir, self.max_restarts, self.backoff_s, hook)
