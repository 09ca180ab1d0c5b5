"""Time the hand-written tcgen05 bf16 GEMMs (single-CTA tiles, CTA-pair tiles, CTA pairs with a K split of the
tail wave) against torch.matmul (cuBLAS) on every Llama-3.1-8B linear shape: forward, dgrad and wgrad.

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

SHAPES = [  # (name, M, N, K, a_mn, b_mn, fp32 accumulate into the output)
    ("qkv_fwd", 4096, 6144, 4096, False, False, False),
    ("proj_fwd", 4096, 4096, 4096, False, False, False),
    ("fc1_fwd", 4096, 28672, 4096, False, False, False),
    ("fc2_fwd", 4096, 4096, 14336, False, False, False),
    ("head_fwd", 4096, 128256, 4096, False, False, False),
    ("qkv_dgrad", 4096, 4096, 6144, False, True, False),
    ("proj_dgrad", 4096, 4096, 4096, False, True, False),
    ("fc1_dgrad", 4096, 4096, 28672, False, True, False),
    ("fc2_dgrad", 4096, 14336, 4096, False, True, False),
    ("head_dgrad", 4096, 4096, 128256, False, True, False),
    ("qkv_wgrad", 6144, 4096, 4096, True, True, True),
    ("proj_wgrad", 4096, 4096, 4096, True, True, True),
    ("fc1_wgrad", 28672, 4096, 4096, True, True, True),
    ("fc2_wgrad", 4096, 14336, 4096, True, True, True),
    ("head_wgrad", 128256, 4096, 4096, True, True, True),
    ("square_8k", 8192, 8192, 8192, False, False, False),
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
    ap.add_argument("--only", default=None, help="comma-separated shape names")
    args = ap.parse_args()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    rows = []
    variants = [("single", False, 1), ("pair", True, 1), ("pair_split", True, 4)]
    only = set(args.only.split(",")) if args.only else None
    for name, M, N, K, a_mn, b_mn, acc in SHAPES:
        if only and name not in only:
            continue
        a = (torch.randn((K, M) if a_mn else (M, K), device="cuda") * 0.5).to(torch.bfloat16)
        b = (torch.randn((K, N) if b_mn else (N, K), device="cuda") * 0.5).to(torch.bfloat16)
        out = torch.zeros(M, N, device="cuda", dtype=torch.float32 if acc else torch.bfloat16)
        am = a.t() if a_mn else a
        bm = b if b_mn else b.t()
        fl = 2.0 * M * N * K
        ref = torch.matmul(am, bm)
        row = {"name": name, "M": M, "N": N, "K": K}
        for vname, pair, slices in variants:
            Fn.set_pair_gemm(pair, slices)
            ours = lambda: Fn.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out, accumulate=acc)
            t, best = time_fn(ours, args.iters, flush)
            out.zero_()
            got = Fn.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out, accumulate=acc)
            err = ((got.float() - ref.float()).norm() / ref.float().norm()).item()
            row[vname + "_ms"] = t
            row[vname + "_tflops"] = fl / t / 1e9
            row[vname + "_rel_err"] = err
        if acc:
            lib = lambda: out.add_(torch.matmul(am, bm))      # what the library arm does for a weight gradient
        else:
            lib = lambda: torch.matmul(am, bm, out=out)
        t_lib, _ = time_fn(lib, args.iters, flush)
        row["cublas_ms"] = t_lib
        row["cublas_tflops"] = fl / t_lib / 1e9
        if acc:
            out_bf = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
            t_mm, _ = time_fn(lambda: torch.matmul(am, bm, out=out_bf), args.iters, flush)
            row["cublas_mm_only_tflops"] = fl / t_mm / 1e9
            del out_bf
        row["best_vs_cublas"] = max(row[v + "_tflops"] for v, _, _ in variants) / row["cublas_tflops"]
        rows.append(row)
        print(json.dumps({k: (round(v, 4) if isinstance(v, float) else v) for k, v in row.items()}), flush=True)
        del a, b, out, ref
    Fn.set_pair_gemm(True, 4)
    print("status word:", _lib.read_status())
    if args.out:
        with open(args.out, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
