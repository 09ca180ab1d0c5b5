"""Quantisation configurations (reference ``utils/quantization_config.py:204-595``)."""
from ..modules.quantizers import AutoQuantizationConfig, Fp8BlockConfig, PtqConfig, QuantizationConfig, RtnConfig, SmoothQuantConfig  # noqa: F401

__all__ = ["AutoQuantizationConfig", "Fp8BlockConfig", "PtqConfig", "QuantizationConfig", "RtnConfig", "SmoothQuantConfig"]
