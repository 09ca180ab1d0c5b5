#!/usr/bin/env python
"""Sustained throughput of the GEMM kernels under the board power cap, with clocks, power and energy per PFLOP.

A B200 training step runs at the 1 kW cap (``sw_power_cap``): the SM clock settles where the kernels' power draw meets
the cap, so what decides the step time is the energy a kernel spends per FLOP, not its speed at boost clocks. A burst
benchmark (a few launches after an idle gap) does not see that. This script loops one kernel for several seconds, samples
``nvidia-smi`` (SM clock, power draw) ten times a second and reports TFLOP/s, TFLOP/s per GHz and joules per PFLOP over
the settled part of the run, for this repository's CTA-pair GEMM at several raster bands and for cuBLAS.

    python benchmarks/bench_sustained_power.py --tokens 8192 --seconds 3 --out sustained.json

It reads clocks and power only; it changes no GPU setting."""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mindformers_b200.ops import _lib  # noqa: E402
from mindformers_b200.ops import functional as Fn  # noqa: E402


def _sample(stop, out, index):
    while not stop.is_set():
        r = subprocess.run(["nvidia-smi", "--query-gpu=clocks.sm,power.draw", "--format=csv,noheader,nounits", "-i", str(index)],
                           capture_output=True, text=True).stdout.strip().split(",")
        try:
            out.append((float(r[0]), float(r[1])))
        except (ValueError, IndexError):
            pass
        time.sleep(0.1)


def run(name, fn, flops, seconds):
    for _ in range(5):
        fn()
    torch.cuda.synchronize()
    stop, samples = threading.Event(), []
    th = threading.Thread(target=_sample, args=(stop, samples, torch.cuda.current_device()))
    th.start()
    n = 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    e0.record()
    while time.time() - t0 < seconds:
        for _ in range(20):
            fn()
        n += 20
        torch.cuda.synchronize()
    e1.record()
    torch.cuda.synchronize()
    stop.set()
    th.join()
    ms = e0.elapsed_time(e1) / n
    tail = samples[len(samples) // 3:] or [(float("nan"), float("nan"))]
    mhz = statistics.median(c for c, _ in tail)
    watts = statistics.mean(p for _, p in tail)
    row = {"case": name, "ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1), "sm_mhz": mhz, "power_w": round(watts, 1),
           "tflops_per_ghz": round(flops / ms / 1e9 / mhz * 1000, 1),
           "joule_per_pflop": round(watts * ms / 1e3 / (flops / 1e15), 2)}
    print(json.dumps(row), flush=True)
    return row


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--seconds", type=float, default=3.0)
    ap.add_argument("--bands", default="8,16,0", help="raster bands of the CTA-pair GEMM to time (0 = chosen by the launcher)")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    lib = _lib.get_lib()
    T = args.tokens
    rows = []
    for (N, K, tag) in [(14336 * 2, 4096, "fc1"), (6144, 4096, "qkv"), (4096, 14336, "fc2")]:
        x = (torch.randn(T, K, device="cuda") * 0.5).to(torch.bfloat16)
        w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
        flops = 2.0 * T * N * K
        for band in [int(b) for b in args.bands.split(",")]:
            lib.mfb_gemm_pair_set_band(band)
            rows.append(run(f"pair_{tag}_band{band}", lambda: Fn.gemm(x, w), flops, args.seconds))
        lib.mfb_gemm_pair_set_band(0)
        rows.append(run(f"cublas_{tag}", lambda: torch.matmul(x, w.t()), flops, args.seconds))
        g = (torch.randn(T, N, device="cuda") * 0.1).to(torch.bfloat16)
        acc = torch.zeros(N, K, device="cuda")
        rows.append(run(f"pair_wgrad_{tag}", lambda: Fn.gemm(g, x, a_mn=True, b_mn=True, out=acc, accumulate=True), flops,
                        args.seconds))
        rows.append(run(f"cublas_wgrad_{tag}", lambda: acc.add_(torch.matmul(g.t(), x)), flops, args.seconds))
    if args.out:
        with open(args.out, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
