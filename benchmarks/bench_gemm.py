"""Time the hand-written tcgen05 bf16 GEMM against torch.matmul (cuBLAS) on Llama-3.1-8B shapes.

Usage: python benchmarks/bench_gemm.py [--iters 20] [--out FILE.json]
Timing: CUDA events, 3 warm-up runs, L2 flushed by writing a 256 MiB buffer between iterations.
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mindformers_b200.ops import functional as Fn  # noqa: E402
from mindformers_b200.ops import _lib  # noqa: E402

SHAPES = [  # (name, M, N, K, a_mn, b_mn)
    ("qkv_fwd", 4096, 6144, 4096, False, False),
    ("fc1_fwd", 4096, 28672, 4096, False, False),
    ("fc2_fwd", 4096, 4096, 14336, False, False),
    ("proj_fwd", 4096, 4096, 4096, False, False),
    ("fc1_dgrad", 4096, 4096, 28672, False, True),
    ("fc1_wgrad", 28672, 4096, 4096, True, True),
    ("head_fwd", 4096, 128256, 4096, False, False),
    ("square_8k", 8192, 8192, 8192, False, False),
]


def time_fn(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.fill_(1.0)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts) // 2], ts[0]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    rows = []
    for name, M, N, K, a_mn, b_mn in SHAPES:
        a = torch.randn((K, M) if a_mn else (M, K), device="cuda", dtype=torch.bfloat16)
        b = torch.randn((K, N) if b_mn else (N, K), device="cuda", dtype=torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        am = a.t() if a_mn else a
        bm = b if b_mn else b.t()
        ours = lambda: Fn.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out)
        lib = lambda: torch.matmul(am, bm, out=out)
        t_ours, b_ours = time_fn(ours, args.iters, flush)
        t_lib, b_lib = time_fn(lib, args.iters, flush)
        ref = torch.matmul(am, bm)
        got = Fn.gemm(a, b, a_mn=a_mn, b_mn=b_mn)
        err = ((got.float() - ref.float()).norm() / ref.float().norm()).item()
        fl = 2.0 * M * N * K
        rows.append({"name": name, "M": M, "N": N, "K": K, "ours_ms": t_ours, "ours_best_ms": b_ours,
                     "cublas_ms": t_lib, "cublas_best_ms": b_lib, "ours_tflops": fl / t_ours / 1e9,
                     "cublas_tflops": fl / t_lib / 1e9, "rel_err_vs_cublas": err})
        print(rows[-1], flush=True)
    print("status word:", _lib.read_status())
    if args.out:
        with open(args.out, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
