"""Time the hand-written tcgen05 flash attention (forward and backward) against PyTorch SDPA.

Usage: python benchmarks/bench_attention.py [--iters 10] [--out FILE.json]
Shapes: causal self-attention of Llama-3.1-8B (32 q heads / 8 kv heads, head dim 128) at several
sequence lengths. Timing: CUDA events, 3 warm-up runs, L2 flushed between iterations.
"""
import argparse
import json
import os
import sys

import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mindformers_b200.ops import attention as A  # noqa: E402
from mindformers_b200.ops import _lib  # noqa: E402


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
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--out", default=None)
    ap.add_argument("--probes", type=int, default=0, help="also time the backward kernel with its timing probes set")
    ap.add_argument("--poly", type=int, default=0, help="quarters of the exponentials on the FMA pipe for the headline rows")
    args = ap.parse_args()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    rows = []
    for B, S, nq, nkv in [(1, 4096, 32, 8), (4, 4096, 32, 8), (1, 16384, 32, 8), (1, 4096, 16, 4)]:
        hd = 128
        packed = (torch.randn(B * S, nq + 2 * nkv, hd, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
        q4 = packed[:, :nq].reshape(B, S, nq, hd)
        k4 = packed[:, nq:nq + nkv].reshape(B, S, nkv, hd)
        v4 = packed[:, nq + nkv:].reshape(B, S, nkv, hd)
        g = torch.randn(B * S, nq * hd, device="cuda", dtype=torch.bfloat16) * 0.1

        def ours_fwd():
            with torch.no_grad():
                return A.flash_attention_packed(packed, B, S, nq, nkv, True)

        def sdpa_fwd():
            with torch.no_grad():
                return F.scaled_dot_product_attention(q4.transpose(1, 2), k4.transpose(1, 2), v4.transpose(1, 2),
                                                      is_causal=True, enable_gqa=True)

        def ours_fb():
            packed.grad = None
            A.flash_attention_packed(packed, B, S, nq, nkv, True).backward(g)

        def sdpa_fb():
            packed.grad = None
            o = F.scaled_dot_product_attention(q4.transpose(1, 2), k4.transpose(1, 2), v4.transpose(1, 2),
                                               is_causal=True, enable_gqa=True)
            o.transpose(1, 2).reshape(B * S, nq * hd).backward(g)

        fl_fwd = 4.0 * B * nq * S * S * hd / 2
        lib = _lib.get_lib()
        variants = {}
        lib.mfb_flash_attn_set_fwd_variant(1)              # one query tile per CTA
        variants["one_tile"] = fl_fwd / time_fn(ours_fwd, args.iters, flush) / 1e9
        lib.mfb_flash_attn_set_fwd_variant(2)              # two query tiles per CTA, 0..2 quarters of exp2 on the FMA pipe
        for poly in range(3):
            lib.mfb_flash_attn_fwd2_set_poly(poly)
            variants[f"two_tiles_poly{poly}"] = fl_fwd / time_fn(ours_fwd, args.iters, flush) / 1e9
        lib.mfb_flash_attn_fwd2_set_poly(args.poly)
        t1, t2 = time_fn(ours_fwd, args.iters, flush), time_fn(sdpa_fwd, args.iters, flush)
        t3, t4 = time_fn(ours_fb, args.iters, flush), time_fn(sdpa_fb, args.iters, flush)
        probes = {}
        if args.probes and hasattr(lib, "mfb_flash_attn_bwd2_set_probe"):
            # where the backward kernel's time goes (results are wrong while a probe is set): 1 = the dQ drain drops its
            # staging and reduce-add, 2 = the compute warpgroups drop the exponentials, 3 = both
            for bits in (1, 2, 3):
                lib.mfb_flash_attn_bwd2_set_probe(bits)
                probes[f"fwd_bwd_ms_probe{bits}"] = time_fn(ours_fb, args.iters, flush)
            lib.mfb_flash_attn_bwd2_set_probe(0)
        rows.append({"B": B, "S": S, "nq": nq, "nkv": nkv, "ours_fwd_ms": t1, "sdpa_fwd_ms": t2,
                     "ours_fwd_tflops": fl_fwd / t1 / 1e9, "sdpa_fwd_tflops": fl_fwd / t2 / 1e9,
                     "ours_fwd_bwd_ms": t3, "sdpa_fwd_bwd_ms": t4,
                     "ours_fwd_bwd_tflops": 3.5 * fl_fwd / t3 / 1e9, "sdpa_fwd_bwd_tflops": 3.5 * fl_fwd / t4 / 1e9,
                     "fwd_variants_tflops": variants, **probes})
        print(rows[-1], flush=True)
    print("status word:", _lib.read_status())
    if args.out:
        with open(args.out, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
