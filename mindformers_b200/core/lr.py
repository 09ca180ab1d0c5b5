"""Learning-rate schedules.

Same catalogue and formulas as the reference's ``core/lr/lr_schedule.py`` (:76-936): linear warm-up from
``warmup_lr_init`` over ``warmup_steps`` (or ``warmup_ratio · total_steps``), then the named decay.
Schedules are callables ``step -> lr`` with steps counted from 1 (the optimizer increments ``global_step``
before the lookup, reference ``adamw.py:190-191``). ``total_steps=-1`` is filled in by the trainer.
"""
from __future__ import annotations

import math
from typing import List, Optional

from ..tools.register import MindFormerModuleType, MindFormerRegister


class _Schedule:
    def __init__(self, learning_rate: float, warmup_steps: Optional[int] = None, warmup_lr_init: float = 0.0,
                 warmup_ratio: Optional[float] = None, total_steps: int = -1, **unused):
        self.learning_rate = float(learning_rate)
        self.warmup_lr_init = float(warmup_lr_init)
        self.total_steps = int(total_steps) if total_steps is not None else -1
        if warmup_ratio is not None:
            if not 0.0 <= warmup_ratio <= 1.0:
                raise ValueError("warmup_ratio must lie in [0, 1]")
            self._warmup_ratio = warmup_ratio
            self.warmup_steps = int(self.total_steps * warmup_ratio) if self.total_steps > 0 else 0
        else:
            self._warmup_ratio = None
            self.warmup_steps = int(warmup_steps or 0)

    def set_total_steps(self, total_steps: int):
        self.total_steps = int(total_steps)
        if self._warmup_ratio is not None:
            self.warmup_steps = int(self.total_steps * self._warmup_ratio)
        self._on_total_steps()

    def _on_total_steps(self):
        pass

    def _warm(self, step: int) -> Optional[float]:
        if self.warmup_steps > 0 and step <= self.warmup_steps:
            frac = step / self.warmup_steps
            return self.warmup_lr_init + (self.learning_rate - self.warmup_lr_init) * frac
        return None

    def decay(self, step: int) -> float:
        return self.learning_rate

    def __call__(self, step: int) -> float:
        step = max(int(step), 0)
        w = self._warm(step)
        return w if w is not None else self.decay(step)


@MindFormerRegister.register(MindFormerModuleType.LR)
class ConstantWarmUpLR(_Schedule):
    """Warm up, then stay at ``learning_rate``."""


@MindFormerRegister.register(MindFormerModuleType.LR)
class LinearWithWarmUpLR(_Schedule):
    """Warm up, then decay linearly to ``lr_end`` (0 by default) at ``total_steps``."""

    def __init__(self, learning_rate, total_steps=-1, lr_end: float = 0.0, **kw):
        super().__init__(learning_rate, total_steps=total_steps, **kw)
        self.lr_end = lr_end

    def decay(self, step):
        span = max(1, self.total_steps - self.warmup_steps)
        frac = max(0.0, (self.total_steps - step) / span)
        return self.lr_end + (self.learning_rate - self.lr_end) * frac


@MindFormerRegister.register(MindFormerModuleType.LR)
class CosineWithWarmUpLR(_Schedule):
    """Warm up, then ``lr_end + (lr - lr_end)·max(0, ½(1 + cos(π·2·num_cycles·progress)))``."""

    def __init__(self, learning_rate, total_steps=-1, num_cycles: float = 0.5, lr_end: float = 0.0,
                 decay_steps: Optional[int] = None, decay_ratio: Optional[float] = None, **kw):
        super().__init__(learning_rate, total_steps=total_steps, **kw)
        self.num_cycles, self.lr_end = num_cycles, lr_end
        self._decay_steps, self._decay_ratio = decay_steps, decay_ratio

    @property
    def decay_steps(self):
        if self._decay_steps:
            return self._decay_steps
        if self._decay_ratio:
            return max(1, int(self.total_steps * self._decay_ratio))
        return max(1, self.total_steps - self.warmup_steps)

    def decay(self, step):
        progress = min(1.0, (step - self.warmup_steps) / self.decay_steps)
        pct = max(0.0, 0.5 * (1.0 + math.cos(math.pi * self.num_cycles * 2.0 * progress)))
        return self.lr_end + (self.learning_rate - self.lr_end) * pct


@MindFormerRegister.register(MindFormerModuleType.LR)
class CosineWithRestartsAndWarmUpLR(CosineWithWarmUpLR):
    """Cosine with ``num_cycles`` hard restarts."""

    def __init__(self, learning_rate, total_steps=-1, num_cycles: float = 1.0, **kw):
        super().__init__(learning_rate, total_steps=total_steps, num_cycles=num_cycles, **kw)

    def decay(self, step):
        progress = min(1.0, (step - self.warmup_steps) / self.decay_steps)
        if progress >= 1.0:
            return self.lr_end
        pct = 0.5 * (1.0 + math.cos(math.pi * ((self.num_cycles * progress) % 1.0)))
        return self.lr_end + (self.learning_rate - self.lr_end) * pct


@MindFormerRegister.register(MindFormerModuleType.LR)
class PolynomialWithWarmUpLR(_Schedule):
    """Linear warm-up, then polynomial decay of degree ``power`` to ``lr_end`` at ``total_steps`` (reference
    ``core/lr/lr_schedule.py``)."""

    def __init__(self, learning_rate, total_steps=-1, lr_end: float = 1e-7, power: float = 1.0, **kw):
        super().__init__(learning_rate, total_steps=total_steps, **kw)
        self.lr_end, self.power = lr_end, power

    def decay(self, step):
        if step >= self.total_steps:
            return self.lr_end
        span = max(1, self.total_steps - self.warmup_steps)
        remaining = 1.0 - (step - self.warmup_steps) / span
        return (self.learning_rate - self.lr_end) * remaining ** self.power + self.lr_end


@MindFormerRegister.register(MindFormerModuleType.LR)
class WarmUpStableDecayLR(_Schedule):
    """Warm up, hold, then decay linearly to ``lr_end`` over the last ``decay_steps`` (or ``decay_ratio``)."""

    def __init__(self, learning_rate, total_steps=-1, lr_end: float = 1e-7, decay_start_steps: Optional[int] = None,
                 decay_steps: Optional[int] = None, decay_ratio: Optional[float] = None, **kw):
        super().__init__(learning_rate, total_steps=total_steps, **kw)
        self.lr_end = lr_end
        self._start, self._dsteps, self._dratio = decay_start_steps, decay_steps, decay_ratio

    def decay(self, step):
        if self._start is not None:
            start = self._start
            length = max(1, self.total_steps - start)
        else:
            length = self._dsteps or max(1, int(self.total_steps * (self._dratio or 0.1)))
            start = self.total_steps - length
        if step <= start:
            return self.learning_rate
        frac = min(1.0, (step - start) / length)
        return self.learning_rate + (self.lr_end - self.learning_rate) * frac


@MindFormerRegister.register(MindFormerModuleType.LR)
class ConstantWithCoolDownLR(_Schedule):
    """DeepSeek-V3 style: warm up, keep ``learning_rate`` for ``keep_steps``, cosine down to ``final_lr`` over
    ``decay_steps``, then hold ``final_lr``."""

    def __init__(self, learning_rate, total_steps=-1, keep_steps: int = 0, decay_steps: Optional[int] = None,
                 decay_ratio: Optional[float] = None, final_steps: int = 0, lr_end1: Optional[float] = None,
                 lr_end2: Optional[float] = None, num_cycles: float = 0.5, **kw):
        super().__init__(learning_rate, total_steps=total_steps, **kw)
        self.keep_steps, self._dsteps, self._dratio = keep_steps, decay_steps, decay_ratio
        self.final_steps, self.num_cycles = final_steps, num_cycles
        self.lr_end1 = lr_end1 if lr_end1 is not None else 0.0
        self.lr_end2 = lr_end2 if lr_end2 is not None else self.lr_end1

    def decay(self, step):
        s = step - self.warmup_steps
        if s <= self.keep_steps:
            return self.learning_rate
        dsteps = self._dsteps or max(1, int(self.total_steps * (self._dratio or 0.0)) or
                                     self.total_steps - self.warmup_steps - self.keep_steps - self.final_steps)
        s -= self.keep_steps
        if s <= dsteps:
            pct = 0.5 * (1.0 + math.cos(math.pi * 2 * self.num_cycles * s / dsteps))
            return self.lr_end1 + (self.learning_rate - self.lr_end1) * pct
        return self.lr_end2


@MindFormerRegister.register(MindFormerModuleType.LR)
class CosineAnnealingLR(_Schedule):
    """PyTorch ``CosineAnnealingLR`` closed form with period ``2·t_max``."""

    def __init__(self, base_lr, t_max: int, eta_min: float = 0.0, **kw):
        super().__init__(base_lr, **kw)
        self.t_max, self.eta_min = t_max, eta_min

    def decay(self, step):
        return self.eta_min + (self.learning_rate - self.eta_min) * (1 + math.cos(math.pi * step / self.t_max)) / 2


@MindFormerRegister.register(MindFormerModuleType.LR)
class CosineAnnealingWarmRestarts(_Schedule):
    """Cosine annealing restarted every ``t_0 * t_mult^i`` steps (SGDR)."""

    def __init__(self, base_lr, t_0: int, t_mult: int = 1, eta_min: float = 0.0, **kw):
        super().__init__(base_lr, **kw)
        if t_0 <= 0 or t_mult < 1:
            raise ValueError("t_0 must be positive and t_mult >= 1")
        self.t_0, self.t_mult, self.eta_min = t_0, t_mult, eta_min

    def decay(self, step):
        t, period = step, self.t_0
        if self.t_mult == 1:
            t = step % self.t_0
        else:
            n = int(math.log(step / self.t_0 * (self.t_mult - 1) + 1, self.t_mult)) if step >= self.t_0 else 0
            t = step - self.t_0 * (self.t_mult ** n - 1) // (self.t_mult - 1)
            period = self.t_0 * self.t_mult ** n
        return self.eta_min + (self.learning_rate - self.eta_min) * (1 + math.cos(math.pi * t / period)) / 2


@MindFormerRegister.register(MindFormerModuleType.LR)
class LearningRateWiseLayer:
    """Wraps a schedule with a per-layer scale (layer-wise lr decay)."""

    def __init__(self, base_lr, lr_scale: float):
        self.base_lr, self.lr_scale = base_lr, lr_scale

    def __call__(self, step):
        return self.lr_scale * self.base_lr(step)


def build_lr(config: Optional[dict] = None, default_args: Optional[dict] = None, **kwargs):
    """Build a schedule from ``{"type": ..., ...}`` (or return a float learning rate unchanged)."""
    if config is None and not kwargs:
        return None
    if isinstance(config, (int, float)):
        return float(config)
    cfg = dict(config or {})
    cfg.update(kwargs)
    if "type" not in cfg:
        return float(cfg["learning_rate"])
    return MindFormerRegister.get_instance_from_cfg(cfg, MindFormerModuleType.LR, default_args=default_args)


from .._submodules import alias_children as _alias_children  # noqa: E402

_alias_children(__name__, ['lr_schedule', 'build_lr'])
