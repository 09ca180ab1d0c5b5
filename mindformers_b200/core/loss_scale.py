"""Loss-scale managers for fp16 training (``wrapper/adaptive_loss_scale.py:64``, ``DynamicLossScaleUpdateCell``); bf16
configurations use a fixed scale of 1 and never touch these."""
from __future__ import annotations

from typing import List

from ..tools.register.register import MindFormerModuleType, MindFormerRegister


@MindFormerRegister.register(MindFormerModuleType.WRAPPER)
class DynamicLossScaleUpdateCell:
    """Halve on overflow, double after ``scale_window`` clean steps."""

    def __init__(self, loss_scale_value: float = 65536.0, scale_factor: float = 2.0, scale_window: int = 1000, **kw):
        self.scale, self.factor, self.window = float(loss_scale_value), float(scale_factor), int(scale_window)
        self.good_steps = 0

    def update(self, overflow: bool) -> float:
        if overflow:
            self.scale = max(self.scale / self.factor, 1.0)
            self.good_steps = 0
        else:
            self.good_steps += 1
            if self.good_steps >= self.window:
                self.scale *= self.factor
                self.good_steps = 0
        return self.scale


@MindFormerRegister.register(MindFormerModuleType.WRAPPER)
class AdaptiveLossScaleUpdateCell(DynamicLossScaleUpdateCell):
    """Window that adapts itself: after each overflow the next (shorter) window of ``window_list`` is used, so the scale
    recovers quickly at first; ``max_scale_window`` clean growth periods move back to longer windows."""

    def __init__(self, loss_scale_value: float = 65536.0, scale_factor: float = 2.0, scale_window: int = 1000,
                 max_scale_window: int = 1000, min_scale_window: int = 20, **kw):
        super().__init__(loss_scale_value, scale_factor, scale_window)
        wins: List[int] = []
        w = max_scale_window
        while w >= min_scale_window:
            wins.append(w)
            w //= 2
        self.windows = wins or [scale_window]
        self.idx = 0
        self.window = self.windows[0]
        self.grow_count = 0

    def update(self, overflow: bool) -> float:
        if overflow:
            self.idx = min(self.idx + 1, len(self.windows) - 1)
            self.window = self.windows[self.idx]
            self.grow_count = 0
            return super().update(True)
        before = self.scale
        out = super().update(False)
        if out > before:
            self.grow_count += 1
            if self.grow_count >= 2 and self.idx > 0:
                self.idx -= 1
                self.window = self.windows[self.idx]
                self.grow_count = 0
        return out
