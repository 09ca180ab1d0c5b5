"""Post-training quantisation of linear layers (``mindformers/modules/quantizers``, ``utils/quantization_config.py``:
RTN / PTQ / SmoothQuant configurations for int8 / int4 weights, int8 activations and int8 KV cache; the reference hands
the work to the Golden-Stick package). Implemented here:

* ``RtnConfig``: round-to-nearest weight-only int8 or int4 (per output channel or per group), de-quantised on the fly;
* ``PtqConfig`` / ``SmoothQuantConfig``: W8A8 with per-token dynamic activation scales; SmoothQuant first migrates
  activation outliers into the weights with ``s_j = max|x_j|^α / max|w_j|^(1-α)`` from calibration statistics;
* ``Fp8BlockConfig``: block-scaled e4m3 weights (128 x 128) run by the fp8 tcgen05 GEMM;
* ``quantize_kv_int8`` / ``dequantize_kv_int8`` for an int8 KV cache with per-token-per-head scales.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as Fn
from ..parallel.layers.tensor_parallel import ColumnParallelLinear, LinearNoTP, RowParallelLinear


@dataclass
class QuantizationConfig:
    """Base quantisation settings (reference ``utils/quantization_config.py:67``): ``quant_method``, weight / activation
    / KV-cache dtypes, modules to skip."""

    quant_method: str = "rtn"
    modules_to_not_convert: Optional[Iterable[str]] = None


@dataclass
class RtnConfig(QuantizationConfig):
    """Round-to-nearest weight-only quantisation (int8 / int4, per channel or per group)."""

    quant_method: str = "rtn"
    weight_dtype: str = "int8"          # int8 | int4
    group_size: int = 0                 # 0 = one scale per output channel


@dataclass
class PtqConfig(QuantizationConfig):
    """Post-training quantisation: int8 weights and activations with calibrated per-channel scales, optional int8 KV
    cache."""

    quant_method: str = "ptq"
    weight_dtype: str = "int8"
    activation_dtype: str = "int8"
    kvcache_dtype: Optional[str] = None


@dataclass
class SmoothQuantConfig(PtqConfig):
    """SmoothQuant W8A8: activation outliers migrated into the weights by a per-channel smoothing factor ``alpha``."""

    quant_method: str = "smooth_quant"
    alpha: float = 0.5


@dataclass
class Fp8BlockConfig(QuantizationConfig):
    """Block-scaled fp8 (e4m3) weights with one scale per 128 x 128 block, activations per 1 x 128 block (the
    DeepSeek-V3 checkpoint format)."""

    quant_method: str = "fp8"
    fmt: str = "e4m3"
    weight_block_size: tuple = (128, 128)


def _qrange(dtype: str):
    return (-8, 7) if dtype == "int4" else (-128, 127)


def quantize_weight_rtn(w: torch.Tensor, dtype: str = "int8", group_size: int = 0):
    """``w [out, in]`` → ``(int8 tensor holding the codes, scale [out, groups])``."""
    lo, hi = _qrange(dtype)
    out_f, in_f = w.shape
    g = group_size if group_size and in_f % group_size == 0 else in_f
    wg = w.float().reshape(out_f, in_f // g, g)
    scale = wg.abs().amax(-1, keepdim=True).clamp_min(1e-8) / hi
    q = torch.round(wg / scale).clamp(lo, hi).to(torch.int8).reshape(out_f, in_f)
    return q, scale.squeeze(-1)


def dequantize_weight(q: torch.Tensor, scale: torch.Tensor, dtype=torch.bfloat16):
    out_f, in_f = q.shape
    groups = scale.shape[1]
    return (q.float().reshape(out_f, groups, in_f // groups) * scale.unsqueeze(-1)).reshape(out_f, in_f).to(dtype)


class QuantLinear(nn.Module):
    """Drop-in for a (column / row / plain) linear layer; returns ``(y, bias)`` like the layer it replaces."""

    def __init__(self, base: nn.Module, cfg: QuantizationConfig, act_absmax: Optional[torch.Tensor] = None):
        super().__init__()
        self.base_kind = type(base).__name__
        self.cfg = cfg
        self.base = base
        w = base.weight.detach()
        self.method = cfg.quant_method
        self.register_buffer("smooth", None)
        if self.method == "fp8":
            q, s = Fn.quantize_weight_128x128(w.float())
            self.register_buffer("qweight", q)
            self.register_buffer("scale", s)
        else:
            if self.method == "smooth_quant" and act_absmax is not None:
                wmax = w.float().abs().amax(0).clamp_min(1e-5)
                s = (act_absmax.float().clamp_min(1e-5) ** cfg.alpha / wmax ** (1 - cfg.alpha)).clamp_min(1e-5)
                self.register_buffer("smooth", s)
                w = w.float() * s
            q, s = quantize_weight_rtn(w.float(), getattr(cfg, "weight_dtype", "int8"), getattr(cfg, "group_size", 0))
            self.register_buffer("qweight", q)
            self.register_buffer("scale", s)
        self.act_int8 = getattr(cfg, "activation_dtype", None) == "int8"
        base.weight = None            # the bf16 copy is dropped: the memory saving is the point

    @property
    def weight(self):
        return self.qweight

    def _matmul(self, x):
        if self.method == "fp8":
            return Fn.fp8_linear(x, self.qweight, self.scale)
        if self.act_int8 and self.scale.shape[1] == 1 and self.smooth is not None:
            return Fn.w8a8_linear(x, self.qweight, self.scale[:, 0], smooth=self.smooth)   # division fused into the quantiser
        if self.smooth is not None:
            x = x / self.smooth.to(x.dtype)
        if self.act_int8 and self.scale.shape[1] == 1:
            # W8A8: per-token dynamic activation scales, per-channel weight scales, the product on the integer tensor
            # cores with an int32 accumulator (the fp32 emulation that stood here was exact only for |sum| < 2^24)
            return Fn.w8a8_linear(x, self.qweight, self.scale[:, 0])
        return F.linear(x, dequantize_weight(self.qweight, self.scale, x.dtype))

    def forward(self, x, *a, **kw):
        from ..parallel import mappings as M
        base = self.base
        tp = getattr(base, "tp", 1)
        if isinstance(base, ColumnParallelLinear):
            xin = x
            if tp > 1:
                xin = M.gather_from_sequence_parallel_region(x) if base.sequence_parallel else M.copy_to_tensor_model_parallel_region(x)
            y = self._matmul(xin)
            if base.bias is not None and not base.skip_bias_add:
                y = y + base.bias
            if base.gather_output and tp > 1:
                y = M.gather_from_tensor_model_parallel_region(y)
            return y, (base.bias if base.skip_bias_add else None)
        if isinstance(base, RowParallelLinear):
            y = self._matmul(x)
            if tp > 1 and not base.delay_allreduce:
                y = M.reduce_scatter_to_sequence_parallel_region(y) if base.sequence_parallel else M.reduce_from_tensor_model_parallel_region(y)
            if base.bias is not None and not base.skip_bias_add:
                y = y + base.bias
            return y, (base.bias if base.skip_bias_add else None)
        y = self._matmul(x)
        bias = getattr(base, "bias", None)
        if bias is not None and not getattr(base, "skip_bias_add", False):
            y = y + bias
        return y, None


def collect_activation_absmax(model: nn.Module, batches, forward) -> Dict[str, torch.Tensor]:
    """Per-input-channel ``max |x|`` of every linear layer over calibration batches (for SmoothQuant)."""
    stats: Dict[str, torch.Tensor] = {}
    hooks = []
    for name, m in model.named_modules():
        if isinstance(m, (ColumnParallelLinear, RowParallelLinear, LinearNoTP)):
            def hook(mod, inp, out, name=name):
                x = inp[0].detach().float().reshape(-1, inp[0].shape[-1]).abs().amax(0)
                stats[name] = torch.maximum(stats[name], x) if name in stats else x
            hooks.append(m.register_forward_hook(hook))
    with torch.no_grad():
        for b in batches:
            forward(model, b)
    for h in hooks:
        h.remove()
    return stats


def quantize_model(model: nn.Module, cfg: QuantizationConfig, act_stats: Optional[Dict[str, torch.Tensor]] = None, prefix: str = "") -> int:
    """Replace linear layers in place (inference only); returns the number of converted layers."""
    skip = list(cfg.modules_to_not_convert or ["output_layer", "router"])
    count = 0
    for name, child in list(model.named_children()):
        full = f"{prefix}.{name}" if prefix else name
        if isinstance(child, (ColumnParallelLinear, RowParallelLinear, LinearNoTP)) and child.weight is not None \
                and not any(s in full for s in skip):
            if cfg.quant_method == "fp8" and (child.weight.shape[0] % 128 or child.weight.shape[1] % 128):
                continue
            setattr(model, name, QuantLinear(child, cfg, (act_stats or {}).get(full)))
            count += 1
        elif not isinstance(child, QuantLinear):
            count += quantize_model(child, cfg, act_stats, full)
    return count


def quantize_kv_int8(x: torch.Tensor):
    """``x [..., head_dim]`` → ``(int8, scale [..., 1])`` with one scale per token and head."""
    s = x.float().abs().amax(-1, keepdim=True).clamp_min(1e-8) / 127.0
    return torch.round(x.float() / s).clamp(-128, 127).to(torch.int8), s


def dequantize_kv_int8(q: torch.Tensor, s: torch.Tensor, dtype=torch.bfloat16):
    return (q.float() * s).to(dtype)


# ---------------------------------------------------------------------------------------------------------------
# configuration dict -> config object -> quantised model (reference ``modules/quantizers/auto.py:33-39``)
# ---------------------------------------------------------------------------------------------------------------
_CONFIG_CLASSES = {"rtn": RtnConfig, "ptq": PtqConfig, "smooth_quant": SmoothQuantConfig, "smoothquant": SmoothQuantConfig,
                   "fp8": Fp8BlockConfig}


class AutoQuantizationConfig:
    """``from_dict({"quant_method": "ptq", ...})`` → the configuration class of that method; unknown keys of a
    Hugging Face ``quantization_config`` (for example ``activation_scheme``) are dropped."""

    @staticmethod
    def from_dict(d: dict) -> QuantizationConfig:
        d = dict(d or {})
        method = str(d.get("quant_method", "rtn")).lower()
        if method not in _CONFIG_CLASSES:
            raise ValueError(f"quant_method {method!r} is not one of {sorted(set(_CONFIG_CLASSES))}")
        cls = _CONFIG_CLASSES[method]
        fields = set(cls.__dataclass_fields__)
        kw = {k: v for k, v in d.items() if k in fields}
        kw["quant_method"] = "smooth_quant" if method == "smoothquant" else method
        if "weight_block_size" in kw:
            kw["weight_block_size"] = tuple(kw["weight_block_size"])
        return cls(**kw)


class AutoQuantizer:
    """``AutoQuantizer.from_config(cfg_or_dict).quantize(model)``: applies the method to a built (and loaded) model.
    Block-scaled fp8 goes through the layers' own fp8 path (``inference/fp8.py``), the integer methods through
    ``quantize_model``; ``act_stats`` are the activation maxima of a calibration run for the W8A8 methods."""

    def __init__(self, config: QuantizationConfig):
        self.config = config

    @classmethod
    def from_config(cls, config) -> "AutoQuantizer":
        return cls(config if isinstance(config, QuantizationConfig) else AutoQuantizationConfig.from_dict(config))

    def quantize(self, model: nn.Module, act_stats: Optional[Dict[str, torch.Tensor]] = None) -> int:
        if self.config.quant_method == "fp8":
            from ..inference.fp8 import quantize_model_fp8
            skip = tuple(self.config.modules_to_not_convert or ("output_layer", "embedding", "router", "linear_kvb"))
            stats = quantize_model_fp8(model, skip=skip)
            return int(stats["linear"]) + int(stats["grouped"])
        n = quantize_model(model, self.config, act_stats)
        kv = getattr(self.config, "kvcache_dtype", None)
        if kv and getattr(model, "config", None) is not None:
            model.config.kv_cache_dtype = str(kv)        # picked up when the generation code allocates the paged cache
        return n


from .._submodules import alias_children as _alias_children  # noqa: E402

_alias_children(__name__, ['auto', 'base', 'ptq_quantizer', 'rtn_quantizer', 'smooth_quant_quantizer'])
