"""Accuracy criteria for kernel and module tests.

Reference: ``tests/utils/double_benchmark.py`` ("double benchmark": the device result is compared with a
high-precision golden result *and* with the result of a trusted second implementation; it passes when its error is at
most ``k`` times the error of that implementation on max / mean relative error, root-mean-square error and the count
of badly-off small values, with thresholds per dtype) and ``tests/utils/precision_utils.py:21-64`` (cosine similarity,
mean absolute error and KL divergence checks).

Use: ``golden`` = fp32 / fp64 PyTorch on the CPU, ``baseline`` = the same operator in plain PyTorch at the kernel's
precision (for example a bf16 ``torch.matmul``), ``actual`` = the hand-written kernel. A fixed absolute tolerance
either hides a precision regression or fails on harmless rounding; comparing with what the precision allows does
neither.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch


@dataclass
class DoubleBenchmarkStandard:
    """Thresholds of one dtype: values below ``small_value`` count as "small" and are judged by absolute error
    ``small_value_atol``; the error ratios actual / baseline may be at most the ``*_ratio`` values."""
    dtype: torch.dtype = torch.bfloat16
    small_value: float = 2 ** -10
    small_value_atol: float = 2 ** -12
    max_rel_ratio: float = 10.0
    mean_rel_ratio: float = 2.0
    rmse_ratio: float = 2.0
    small_count_ratio: float = 2.0
    eps: float = 1e-12

    @classmethod
    def for_dtype(cls, dtype: torch.dtype) -> "DoubleBenchmarkStandard":
        if dtype == torch.float16:
            return cls(dtype, 2 ** -11, 2 ** -16)
        if dtype == torch.bfloat16:
            return cls(dtype, 2 ** -10, 2 ** -12)
        if dtype == torch.float32:
            return cls(dtype, 2 ** -14, 2 ** -30)
        if dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
            return cls(dtype, 2 ** -6, 2 ** -8)
        raise ValueError(f"no accuracy standard for {dtype}")


def error_metrics(result: torch.Tensor, golden: torch.Tensor, std: DoubleBenchmarkStandard) -> Dict[str, float]:
    """Max / mean relative error over the values that are not small, RMSE over all, and the number of small values
    whose absolute error exceeds the small-value tolerance."""
    r, g = result.detach().double().flatten().cpu(), golden.detach().double().flatten().cpu()
    if r.shape != g.shape:
        raise ValueError(f"shapes differ: {tuple(result.shape)} vs {tuple(golden.shape)}")
    if not torch.isfinite(r).all():
        return {"max_rel": float("inf"), "mean_rel": float("inf"), "rmse": float("inf"), "small_bad": float(r.numel())}
    small = g.abs() < std.small_value
    big = ~small
    err = (r - g).abs()
    rel = err[big] / g[big].abs()
    return {"max_rel": float(rel.max()) if rel.numel() else 0.0, "mean_rel": float(rel.mean()) if rel.numel() else 0.0,
            "rmse": float(err.pow(2).mean().sqrt()), "small_bad": float((err[small] > std.small_value_atol).sum())}


class DoubleBenchmarkComparator:
    """``check_pass_or_not(actual, baseline, golden)`` → ``(passed, report)``."""

    def __init__(self, standard: Optional[DoubleBenchmarkStandard] = None, dtype: Optional[torch.dtype] = None):
        self.std = standard or DoubleBenchmarkStandard.for_dtype(dtype or torch.bfloat16)

    def check_pass_or_not(self, actual: torch.Tensor, baseline: torch.Tensor, golden: torch.Tensor):
        s = self.std
        a, b = error_metrics(actual, golden, s), error_metrics(baseline, golden, s)
        limits = {"max_rel": s.max_rel_ratio, "mean_rel": s.mean_rel_ratio, "rmse": s.rmse_ratio,
                  "small_bad": s.small_count_ratio}
        report, ok = {}, True
        for key, limit in limits.items():
            floor = 1.0 if key == "small_bad" else s.eps          # a perfect baseline still allows rounding noise
            allowed = limit * max(b[key], floor)
            passed = a[key] <= allowed
            report[key] = {"actual": a[key], "baseline": b[key], "allowed": allowed, "passed": passed}
            ok = ok and passed
        return ok, report


def cosine_similarity(a: torch.Tensor, b: torch.Tensor) -> float:
    x, y = a.detach().double().flatten(), b.detach().double().flatten()
    return float(torch.dot(x, y) / (x.norm() * y.norm() + 1e-30))


def mean_abs_error(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.detach().double() - b.detach().double()).abs().mean())


def kl_divergence(logits_p: torch.Tensor, logits_q: torch.Tensor) -> float:
    """KL(softmax(p) || softmax(q)) averaged over the leading dimensions."""
    lp = torch.log_softmax(logits_p.detach().double(), dim=-1)
    lq = torch.log_softmax(logits_q.detach().double(), dim=-1)
    return float((lp.exp() * (lp - lq)).sum(-1).mean())


def precision_check(actual: torch.Tensor, expected: torch.Tensor, cos_threshold: float = 0.999,
                    l1_threshold: float = 0.01, kl_threshold: Optional[float] = None) -> Dict[str, float]:
    """Raises ``AssertionError`` with the measured figures when a criterion fails; returns them otherwise."""
    out = {"cosine": cosine_similarity(actual, expected), "l1": mean_abs_error(actual, expected)}
    if kl_threshold is not None:
        out["kl"] = kl_divergence(expected, actual)
    bad = [k for k, ok in (("cosine", out["cosine"] >= cos_threshold), ("l1", out["l1"] <= l1_threshold),
                           ("kl", kl_threshold is None or out.get("kl", 0.0) <= kl_threshold)) if not ok]
    if bad:
        raise AssertionError(f"precision check failed on {bad}: {out}")
    return out
