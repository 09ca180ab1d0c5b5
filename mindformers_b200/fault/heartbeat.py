"""Host-side failure detection: every rank publishes a heartbeat to the job's key-value store, a monitor thread on
every rank watches the others and raises ``RankFailure`` in the training loop (between steps) when a peer goes silent
or announces an error.

The reference delegates this to MindSpore's fault-tolerance runtime (``MS_ENABLE_TFT``; ``core/callback/callback.py``
wires only the callbacks); here the mechanism is explicit and runs entirely on the host, so a dead rank is noticed
*before* the next collective is launched and no GPU wait is left hanging: ranks leave only between steps, with none
of their kernels or collectives in flight.
"""
from __future__ import annotations

import threading
import time
from typing import Dict, List, Optional

import torch.distributed as dist


class RankFailure(RuntimeError):
    """Raised between steps when a peer stopped sending heartbeats or reported an error."""

    def __init__(self, ranks: List[int], reason: str):
        super().__init__(f"rank(s) {ranks} failed: {reason}")
        self.ranks, self.reason = ranks, reason


class HeartbeatMonitor:
    """``store``: any ``torch.distributed`` store (TCPStore / FileStore / HashStore for tests)."""

    def __init__(self, store, rank: int, world_size: int, interval: float = 1.0, timeout: float = 10.0, prefix: str = "hb"):
        self.store, self.rank, self.world = store, rank, world_size
        self.interval, self.timeout, self.prefix = interval, timeout, prefix
        self._stop = threading.Event()
        self._failed: Dict[int, str] = {}
        self._lock = threading.Lock()
        self._thread: Optional[threading.Thread] = None
        self._beat = 0
        self._last_seen: Dict[int, tuple] = {}

    # ---- publishing ------------------------------------------------------------------------------
    def _key(self, rank, what="beat"):
        return f"{self.prefix}/{what}/{rank}"

    def beat(self):
        self._beat += 1
        self.store.set(self._key(self.rank), str(self._beat))

    def report_error(self, message: str):
        """Announce that this rank is about to leave (exception in the step loop)."""
        self.store.set(self._key(self.rank, "error"), message[:500])

    # ---- watching ---------------------------------------------------------------------------------
    def _poll(self):
        now = time.monotonic()
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                if self.store.check([self._key(r, "error")]):
                    with self._lock:
                        self._failed[r] = self.store.get(self._key(r, "error")).decode(errors="replace")
                    continue
                val = self.store.get(self._key(r)).decode() if self.store.check([self._key(r)]) else None
            except Exception as e:  # store unreachable: the host of the store is gone
                with self._lock:
                    self._failed[r] = f"store error: {e}"
                continue
            seen = self._last_seen.get(r)
            if val is not None and (seen is None or seen[0] != val):
                self._last_seen[r] = (val, now)
            elif seen is not None and now - seen[1] > self.timeout:
                with self._lock:
                    self._failed[r] = f"no heartbeat for {now - seen[1]:.1f}s"
            elif seen is None:
                self._last_seen[r] = (None, now) if r not in self._last_seen else self._last_seen[r]

    def _run(self):
        while not self._stop.is_set():
            try:
                self.beat()
                self._poll()
            except Exception:  # noqa: BLE001 - never kill the watcher thread
                pass
            self._stop.wait(self.interval)

    def start(self):
        self.beat()
        self._thread = threading.Thread(target=self._run, daemon=True, name="heartbeat")
        self._thread.start()
        return self

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1)

    def failed_ranks(self) -> Dict[int, str]:
        with self._lock:
            return dict(self._failed)

    def check(self):
        """Call between steps: raises ``RankFailure`` if a peer is known to be gone."""
        bad = self.failed_ranks()
        if bad:
            raise RankFailure(sorted(bad), "; ".join(f"{r}: {m}" for r, m in sorted(bad.items())))


class HeartbeatCallback:
    """Trainer callback: beats at every step, checks peers before the next step is launched."""

    def __init__(self, monitor: HeartbeatMonitor):
        self.monitor = monitor

    def on_train_begin(self, ctx):
        self.monitor.start()

    def on_step_begin(self, ctx):
        self.monitor.check()

    def on_step_end(self, ctx):
        self.monitor.beat()

    def on_epoch_end(self, ctx): ...

    def on_train_end(self, ctx):
        self.monitor.stop()

    def on_exception(self, ctx, exc):
        self.monitor.report_error(f"{type(exc).__name__}: {exc}")
        self.monitor.stop()
