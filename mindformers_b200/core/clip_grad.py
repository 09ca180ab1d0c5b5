"""Global-norm gradient clipping for plain ``.grad`` tensors (reference ``core/clip_grad.py:60-101``).

The flat-buffer optimizer clips inside its fused kernel; this class serves optimizers from ``torch.optim``.
"""
from __future__ import annotations

import torch


class ClipGradNorm:
    """Global-norm clipping (reference ``core/clip_grad.py:60-101``): ``norm = sqrt(sum ||g||^2)``, gradients scaled
    by ``min(1, max_norm / (norm + 1e-6))``; returns the gradients and the norm."""

    def __init__(self, max_norm: float = 1.0, use_norm=None):
        self.max_norm = float(max_norm)
        self.use_norm = use_norm

    @torch.no_grad()
    def __call__(self, grads):
        """Returns ``(clipped_grads, global_norm)``; the coefficient ``max_norm/(norm+1e-6)`` applies only when
        the norm reaches ``max_norm``."""
        grads = [g for g in grads if g is not None]
        if self.use_norm is not None:
            norm = torch.as_tensor(self.use_norm, dtype=torch.float32)
        else:
            norm = torch.sqrt(sum((g.float() ** 2).sum() for g in grads)) if grads else torch.zeros(())
        coef = torch.clamp(self.max_norm / (norm + 1e-6), max=1.0)
        return [g * coef.to(g.dtype) for g in grads], norm
