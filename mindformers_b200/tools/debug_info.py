"""Latency breakdown and token-indexed profiling of ``generate()``.

Reference: ``mindformers/tools/debug_info.py`` — ``DetailedLatency`` (timers around pre-processing, the model call and
post-processing of every generation step, :53-112) and ``Profiling`` (a profiler started and stopped at token indices
taken from the environment, :28-46, :115-147), both owned by ``GenerationMixin``.

Timers here are host timers around the three phases; with ``sync=True`` the device is synchronised at every boundary
so that the model phase holds the kernels' time and not just their launch. ``Profiling`` drives ``torch.profiler`` (and
an NVTX range per decode step) between two token indices: ``MF_PROFILE_START_TOKEN`` / ``MF_PROFILE_STOP_TOKEN`` /
``MF_PROFILE_DIR``.
"""
from __future__ import annotations

import os
import time
from collections import defaultdict
from contextlib import contextmanager
from typing import Dict, List, Optional

import torch

PHASES = ("preprocess", "predict", "postprocess")


class DetailedLatency:
    """Per-step wall times of the three phases of a generation step, split into prefill and decode steps."""

    def __init__(self, enabled: Optional[bool] = None, sync: bool = False):
        self.enabled = (os.environ.get("MF_DETAILED_LATENCY", "0") == "1") if enabled is None else bool(enabled)
        self.sync = sync
        self.clear()

    def clear(self):
        self.records: Dict[str, Dict[str, List[float]]] = {"prefill": defaultdict(list), "decode": defaultdict(list)}

    @contextmanager
    def phase(self, name: str, prefill: bool):
        if not self.enabled:
            yield
            return
        if name not in PHASES:
            raise ValueError(f"phase must be one of {PHASES}")
        if self.sync and torch.cuda.is_available():
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        try:
            yield
        finally:
            if self.sync and torch.cuda.is_available():
                torch.cuda.synchronize()
            self.records["prefill" if prefill else "decode"][name].append(time.perf_counter() - t0)

    def summary(self) -> dict:
        """``{stage: {phase: {count, total_ms, mean_ms, max_ms}}}``."""
        out: dict = {}
        for stage, phases in self.records.items():
            out[stage] = {}
            for name in PHASES:
                v = phases.get(name, [])
                if v:
                    out[stage][name] = {"count": len(v), "total_ms": 1e3 * sum(v), "mean_ms": 1e3 * sum(v) / len(v),
                                        "max_ms": 1e3 * max(v)}
        return out

    def print_info(self, log=None):
        from .logger import logger
        log = log or logger
        for stage, phases in self.summary().items():
            for name, s in phases.items():
                log.info("latency %s/%s: %d steps, mean %.3f ms, max %.3f ms, total %.1f ms", stage, name, s["count"],
                         s["mean_ms"], s["max_ms"], s["total_ms"])


class Profiling:
    """Profiler window over generated tokens: starts before token ``start`` is produced, stops after token ``stop``."""

    def __init__(self, start: Optional[int] = None, stop: Optional[int] = None, output_dir: Optional[str] = None,
                 profiler_factory=None):
        env = os.environ
        self.start = int(env["MF_PROFILE_START_TOKEN"]) if start is None and "MF_PROFILE_START_TOKEN" in env else start
        self.stop = int(env["MF_PROFILE_STOP_TOKEN"]) if stop is None and "MF_PROFILE_STOP_TOKEN" in env else stop
        self.output_dir = output_dir or env.get("MF_PROFILE_DIR", "./output/profile_generate")
        self.enabled = self.start is not None and self.stop is not None and self.stop >= self.start
        self._factory = profiler_factory or self._torch_profiler
        self._prof = None
        self.windows = 0

    def _torch_profiler(self):
        acts = [torch.profiler.ProfilerActivity.CPU]
        if torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        os.makedirs(self.output_dir, exist_ok=True)
        return torch.profiler.profile(activities=acts,
                                      on_trace_ready=torch.profiler.tensorboard_trace_handler(self.output_dir))

    def step_begin(self, token_index: int):
        """Call before the model produces token ``token_index`` (0 = the token that prefill yields)."""
        if not self.enabled:
            return
        if token_index == self.start and self._prof is None:
            self._prof = self._factory()
            self._prof.__enter__()
        if self._prof is not None and torch.cuda.is_available():
            torch.cuda.nvtx.range_push(f"generate token {token_index}")

    def step_end(self, token_index: int):
        if not self.enabled or self._prof is None:
            return
        if torch.cuda.is_available():
            torch.cuda.nvtx.range_pop()
        if token_index >= self.stop:
            self._prof.__exit__(None, None, None)
            self._prof = None
            self.windows += 1

    def close(self):
        """Stops a window that generation ended inside of."""
        if self._prof is not None:
            self._prof.__exit__(None, None, None)
            self._prof = None
            self.windows += 1
