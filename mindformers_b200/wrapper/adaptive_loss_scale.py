"""``AdaptiveLossScaleUpdateCell`` (reference ``wrapper/adaptive_loss_scale.py:64``)."""
from ..core.loss_scale import AdaptiveLossScaleUpdateCell, DynamicLossScaleUpdateCell  # noqa: F401

__all__ = ["AdaptiveLossScaleUpdateCell", "DynamicLossScaleUpdateCell"]
