"""Launch one kernel family a few times on a small case (inputs larger than L2, a few hundred MB on the device):
the target of `ncu -k regex:<kernel> -c N`. Usage: python benchmarks/run_kernel_once.py --kernel gemm

Cases: gemm (fc1 forward 4096 x 28672 x 4096, then dgrad and wgrad layouts), fa (forward + backward, S=4096, 32/8
heads), rmsnorm, swiglu, rope, ce (4096 x 128256 logits), adamw (64 M parameters), router (E=128 top-8 and E=256
group-limited), paged (decode attention, 64 sequences of 2048 tokens, block 128), mla (latent-cache decode, 64 x 2304
tokens, both kernel variants), moe (single-rank exchange kernels), fp8 (block-scaled GEMM at prefill sizes against the
bf16 kernel), fp8_decode (64-token GEMMs: 128-row tiles, cluster split-K, weight-on-rows kernel; graph replay, weights
cycled past L2), fp8_moe_decode (32 experts with two tokens each; MFB_BENCH_EXPERTS shrinks it for an ncu capture).
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mindformers_b200.ops import functional as Fn  # noqa: E402
from mindformers_b200.ops import _lib  # noqa: E402


def bf(*shape, scale=0.5):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def gemm():
    x, w = bf(4096, 4096), bf(28672, 4096, scale=0.05)
    for _ in range(3):
        y = Fn.gemm(x, w)                                   # forward  [4096, 28672]
    dy = bf(4096, 28672, scale=0.1)
    for _ in range(3):
        Fn.gemm(dy, w, b_mn=True)                           # dgrad    [4096, 4096]
    out = torch.zeros(28672, 4096, device="cuda")
    for _ in range(3):
        Fn.gemm(dy, x, a_mn=True, b_mn=True, out=out, accumulate=True)   # wgrad, fp32 accumulate
    return y


def fa():
    from mindformers_b200.ops import attention as A
    B, S, nq, nkv = 1, 4096, 32, 8
    packed = bf(B * S, nq + 2 * nkv, 128).requires_grad_()
    g = bf(B * S, nq * 128, scale=0.1)
    for _ in range(3):
        packed.grad = None
        A.flash_attention_packed(packed, B, S, nq, nkv, True).backward(g)


def rmsnorm():
    T, H = 32768, 4096
    x, w = bf(T, H).requires_grad_(), torch.ones(H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    res = bf(T, H)
    dy = bf(T, H, scale=0.1)
    for _ in range(3):
        Fn.rmsnorm(x, w, 1e-5)[0].backward(dy)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    with torch.no_grad():
        ev[0].record()
        for _ in range(5):
            Fn.rmsnorm(x, w, 1e-5)
        ev[1].record()
        for _ in range(5):
            Fn.rmsnorm(x, w, 1e-5, residual=res)
        ev[2].record()
    # backward through the library entry point (the autograd wrapper would add the accumulation into x.grad)
    lib = _lib.get_lib()
    rstd = torch.empty(T, dtype=torch.float32, device="cuda")
    yb = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
    xd = x.detach()
    _lib.check(lib.mfb_rmsnorm_fwd(xd.data_ptr(), 0, w.data_ptr(), yb.data_ptr(), 0, rstd.data_ptr(), T, H, 1e-5,
                                   _lib.stream_ptr()), "fwd")
    dx = torch.empty_like(xd)
    dwf = torch.empty(H, dtype=torch.float32, device="cuda")
    scratch = torch.empty(lib.mfb_rmsnorm_bwd_parts(T) * H, dtype=torch.float32, device="cuda")

    def bwd(dres):
        _lib.check(lib.mfb_rmsnorm_bwd(dy.data_ptr(), xd.data_ptr(), w.data_ptr(), rstd.data_ptr(), _lib.ptr(dres),
                                       dx.data_ptr(), dwf.data_ptr(), 0, 0, scratch.data_ptr(), T, H, _lib.stream_ptr()),
                   "bwd")
    bwd(None)
    bwd(res)
    torch.cuda.synchronize()
    ev2 = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    ev2[0].record()
    for _ in range(5):
        bwd(None)
    ev2[1].record()
    for _ in range(5):
        bwd(res)
    ev2[2].record()
    torch.cuda.synchronize()
    t_b0, t_b1 = ev2[0].elapsed_time(ev2[1]) / 5, ev2[1].elapsed_time(ev2[2]) / 5
    row = T * H * 2
    t_f, t_r = ev[0].elapsed_time(ev[1]) / 5, ev[1].elapsed_time(ev[2]) / 5
    bw = lambda nbytes, ms: nbytes / ms / 1e6 / 6523.7
    print(f"rmsnorm fwd {t_f * 1e3:.1f} us ({bw(2 * row, t_f):.2f} of measured HBM), fwd+residual {t_r * 1e3:.1f} us "
          f"({bw(4 * row, t_r):.2f}), bwd (dx + dw) {t_b0 * 1e3:.1f} us ({bw(3 * row, t_b0):.2f} of the 3 tensors it "
          f"must touch), bwd with residual gradient {t_b1 * 1e3:.1f} us ({bw(4 * row, t_b1):.2f})")

def swiglu():
    x = bf(16384, 2 * 14336).requires_grad_()
    for _ in range(3):
        Fn.swiglu(x).backward(bf(16384, 14336, scale=0.1))


def rope():
    T, heads = 32768, 40
    x = bf(T, heads, 128).requires_grad_()
    inv = 1.0 / (500000.0 ** (torch.arange(0, 128, 2, device="cuda").float() / 128))
    ang = torch.arange(4096, device="cuda").float()[:, None] * inv[None]
    cos, sin = torch.cat([ang, ang], -1).cos(), torch.cat([ang, ang], -1).sin()
    pos = torch.arange(T, device="cuda") % 4096
    for _ in range(3):
        Fn.rope(x, cos, sin, pos, heads, 128, False).backward(bf(T, heads, 128, scale=0.1))
    with torch.no_grad():
        ms = _timed(lambda: Fn.rope(x, cos, sin, pos, heads, 128, False))
    nbytes = 2 * T * heads * 128 * 2
    print(f"rope forward: {ms * 1e3:.1f} us, {nbytes / ms / 1e6:.0f} GB/s ({nbytes / ms / 1e6 / 6523.7 * 100:.0f} % of measured HBM copy bandwidth)")


def ce():
    logits = bf(4096, 128256, scale=1.0).requires_grad_()
    labels = torch.randint(0, 128256, (4096,), device="cuda")
    for _ in range(3):
        Fn.cross_entropy(logits, labels).sum().backward()


def adamw():
    n = 64 * 1024 * 1024
    p = bf(n, scale=0.02)
    lo = torch.zeros(n, dtype=torch.int16, device="cuda")
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    g = torch.randn(n, device="cuda") * 1e-3
    ss = torch.zeros(1, device="cuda")
    for step in range(1, 4):
        Fn.grad_sumsq(g, ss)
        Fn.adamw_step(p, lo, m, v, g, lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=step, sumsq=ss,
                      max_norm=1.0)
    ms = _timed(lambda: Fn.adamw_step(p, lo, m, v, g, lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=5,
                                      sumsq=ss, max_norm=1.0))
    nbytes = n * (4 + 2 * 2 + 2 * 2 + 4 * 2 + 4 * 2)      # grad read; bf16 param, int16 remainder, m, v read + written
    print(f"adamw: {ms * 1e3:.1f} us, {nbytes / ms / 1e6:.0f} GB/s ({nbytes / ms / 1e6 / 6523.7 * 100:.0f} % of measured HBM copy bandwidth)")


def router():
    for E, k, sig, groups, gk in ((128, 8, False, 0, 0), (256, 8, True, 8, 4)):
        logits = (torch.randn(65536, E, device="cuda") * 2).requires_grad_()
        bias = torch.zeros(E, device="cuda") if sig else None
        for _ in range(3):
            p, ids, _ = Fn.router_topk(logits, bias, k, sigmoid=sig, norm=True, scale=1.0, groups=groups, group_topk=gk)
            p.sum().backward()


def paged():
    lib = _lib.get_lib()
    B, ctx, blk, nq, nkv, hd = 64, 2048, 128, 32, 8, 128
    nblocks = B * ctx // blk
    kc, vc = bf(nblocks, blk, nkv, hd), bf(nblocks, blk, nkv, hd)
    q = bf(B, nq, hd)
    out = torch.empty_like(q)
    tables = torch.arange(nblocks, device="cuda", dtype=torch.int32).view(B, ctx // blk).contiguous()
    lens = torch.full((B,), ctx, device="cuda", dtype=torch.int32)
    splits = lib.mfb_paged_decode_splits(B, nkv, blk, ctx // blk)
    scratch = torch.empty(lib.mfb_paged_decode_scratch_bytes(B, nq, hd, splits) // 4, device="cuda")
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    for i in range(4):
        if i == 1:
            ev[0].record()
        rc = lib.mfb_paged_decode_attention(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), tables.data_ptr(), lens.data_ptr(),
                                            out.data_ptr(), scratch.data_ptr(), splits, B, nq, nkv, hd, blk, ctx // blk,
                                            hd ** -0.5, _lib.stream_ptr())
        _lib.check(rc, "paged")
    ev[1].record()
    torch.cuda.synchronize()
    ms = ev[0].elapsed_time(ev[1]) / 3
    kv_bytes = 2 * B * ctx * nkv * hd * 2
    print(f"paged decode: {ms * 1e3:.1f} us, {kv_bytes / ms / 1e6:.0f} GB/s of KV ({kv_bytes / ms / 1e6 / 6523.7 * 100:.0f} % of measured HBM copy bandwidth), splits {splits}")


def mla():
    """MLA decode: 64 sequences of 2304 cached tokens, 16 heads per rank (128 heads over tp 8) and all 128 heads."""
    from mindformers_b200.inference.paged_attention import mla_decode_attention, set_mla_decode_variant
    B, ctx, blk = 64, 2304, 128
    nblocks = B * ctx // blk
    cache = bf(nblocks, blk, 1, 576)
    tables = torch.arange(nblocks, device="cuda", dtype=torch.int32).view(B, ctx // blk).contiguous()
    lens = torch.full((B,), ctx, device="cuda", dtype=torch.int32)

    class Holder:
        pass

    for variant, nh in (("single", 16), ("single", 128), ("cluster", 16), ("cluster", 128)):
        set_mla_decode_variant(variant)
        q = bf(B, nh, 576, scale=0.3)
        h = Holder()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        for i in range(5):
            if i == 2:
                ev[0].record()
            out = mla_decode_attention(q, cache, tables, lens, blk, 192 ** -0.5, h)
        ev[1].record()
        torch.cuda.synchronize()
        ms = ev[0].elapsed_time(ev[1]) / 3
        kv_bytes = B * ctx * 576 * 2
        flops = 2.0 * B * ctx * nh * (576 + 512)
        print(f"mla decode ({variant}) heads={nh}: {ms * 1e3:.1f} us, {kv_bytes / ms / 1e6:.0f} GB/s of latent cache "
              f"({kv_bytes / ms / 1e6 / 6523.7 * 100:.0f} % of measured HBM copy bandwidth), "
              f"{flops / ms / 1e9:.0f} TFLOP/s, status {_lib.read_status()}")
    set_mla_decode_variant("single")


def moe():
    from mindformers_b200.parallel.layers.moe import MoELayer
    from mindformers_b200.parallel.transformer_config import TransformerConfig
    cfg = TransformerConfig(num_layers=1, hidden_size=2048, num_attention_heads=16, ffn_hidden_size=8192, num_moe_experts=16,
                            moe_router_topk=8, moe_ffn_hidden_size=768, params_dtype=torch.bfloat16, compute_dtype=torch.bfloat16)
    cfg.device = "cuda"
    layer = MoELayer(cfg).train()
    x = bf(16384, 2048).requires_grad_()
    for _ in range(3):
        y, _ = layer(x)
        y.float().mean().backward()


def grouped():
    """Grouped expert GEMMs at the Qwen3-30B-A3B shapes of one expert-parallel rank out of 8: 16 local experts, hidden
    2048, expert FFN 768 (fc1 N = 1536, fc2 K = 768), 4096 tokens x top-8 / 8 ranks = 4096 rows on average."""
    E, H, F_ = 16, 2048, 768
    rows_per = [256] * E                              # balanced routing, segments padded to 128
    R = sum(rows_per)
    x = bf(R, H)
    w1 = bf(E, H, 2 * F_, scale=0.05)                 # [E, in, out]
    w2 = bf(E, F_, H, scale=0.05)
    block_group = torch.tensor([e for e, r in enumerate(rows_per) for _ in range(r // 128)], dtype=torch.int32, device="cuda")
    num_blocks = torch.tensor([block_group.numel()], dtype=torch.int32, device="cuda")
    offs = torch.tensor([0] + list(torch.tensor(rows_per).cumsum(0)), dtype=torch.int32, device="cuda")
    for _ in range(3):
        h = Fn.grouped_gemm(x, w1, block_group, num_blocks, b_mn=True)          # fc1  [R, 1536]
    a = bf(R, F_)
    for _ in range(3):
        y = Fn.grouped_gemm(a, w2, block_group, num_blocks, b_mn=True)          # fc2  [R, 2048]
    dw = torch.zeros(E, H, 2 * F_, device="cuda")
    for _ in range(3):
        Fn.grouped_wgrad(x, h, offs, E, dw, accumulate=True)                    # wgrad of fc1
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    ev[0].record()
    for _ in range(10):
        Fn.grouped_gemm(x, w1, block_group, num_blocks, b_mn=True)
    ev[1].record()
    for _ in range(10):
        Fn.grouped_gemm(a, w2, block_group, num_blocks, b_mn=True)
    ev[2].record()
    for _ in range(10):
        Fn.grouped_wgrad(x, h, offs, E, dw, accumulate=True)
    ev[3].record()
    torch.cuda.synchronize()
    for name, i, fl in (("fc1", 0, 2.0 * R * H * 2 * F_), ("fc2", 1, 2.0 * R * F_ * H), ("wgrad fc1", 2, 2.0 * R * H * 2 * F_)):
        ms = ev[i].elapsed_time(ev[i + 1]) / 10
        print(f"grouped {name}: {ms * 1e3:.1f} us, {fl / ms / 1e9:.0f} TFLOP/s")
    return y


def fp8():
    for (M, N, K) in ((4096, 4096, 7168), (8192, 7168, 2048), (4096, 18432, 7168)):
        x = bf(M, K, scale=0.7)
        w = torch.randn(N, K, device="cuda") * 0.05
        wq, sb = Fn.quantize_weight_128x128(w)
        wb = w.to(torch.bfloat16)
        xq, sa = Fn.quantize_act_1x128(x)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        for i in range(6):
            if i == 1:
                ev[0].record()
            Fn.fp8_gemm(xq, sa, wq, sb)
        ev[1].record()
        for i in range(6):
            if i == 1:
                ev[2].record()
            Fn.gemm(x, wb)
        ev[3].record()
        torch.cuda.synchronize()
        t8, t16 = ev[0].elapsed_time(ev[1]) / 5, ev[2].elapsed_time(ev[3]) / 5
        fl = 2.0 * M * N * K
        print(f"fp8 block-scaled {M}x{N}x{K}: {t8 * 1e3:.1f} us = {fl / t8 / 1e9:.0f} TFLOP/s; bf16 kernel {t16 * 1e3:.1f} us = {fl / t16 / 1e9:.0f} TFLOP/s")
        for _ in range(2):
            Fn.quantize_act_1x128(x)


def fp8_decode():
    """Decode-sized fp8 GEMMs (64 tokens): weight streaming with and without the cluster split over K. Several
    copies of the weight are cycled so that every call reads from HBM, not from L2."""
    lib = _lib.get_lib()
    M = 64
    for (N, K, what) in ((7168, 16384, "o_proj, 1 GPU"), (7168, 18432, "dense fc2, 1 GPU"), (1536, 7168, "q_a"),
                         (3072, 1536, "q_b, tp 8"), (7168, 2048, "o_proj, tp 8"), (4608, 7168, "dense fc1, tp 8")):
        copies = max(2, int(400e6 // (N * K)) + 1)
        ws = []
        for _ in range(copies):
            wq, sb = Fn.quantize_weight_128x128(torch.randn(N, K, device="cuda") * 0.05)
            ws.append((wq, sb))
        xq, sa = Fn.quantize_act_1x128(bf(M, K, scale=0.7))
        res = {}
        for mode in ("tile", "split", "decode"):
            # "tile": 128 token rows per tile, one CTA per tile; "split": the same with K split over a cluster;
            # "decode": the weight on the MMA rows (gemm_fp8_decode.cu)
            lib.mfb_gemm_fp8_enable_ksplit(0 if mode == "tile" else 1)
            Fn._FP8_DECODE_KERNEL = mode == "decode"
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            for i in range(copies):
                Fn.fp8_gemm(xq, sa, *ws[i])
            torch.cuda.synchronize()
            # the calls are replayed from a CUDA graph: at these sizes Python would otherwise be the slower side
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for i in range(copies):
                    Fn.fp8_gemm(xq, sa, *ws[i])
            g.replay()
            ev[0].record()
            for _ in range(4):
                g.replay()
            ev[1].record()
            torch.cuda.synchronize()
            res[mode] = ev[0].elapsed_time(ev[1]) / (4 * copies)
        lib.mfb_gemm_fp8_enable_ksplit(1)
        Fn._FP8_DECODE_KERNEL = True
        gbs = N * K / res["decode"] / 1e6
        print(f"fp8 decode {M}x{N}x{K} ({what}): 128-row tiles {res['tile'] * 1e3:.1f} us, with cluster split-K "
              f"{res['split'] * 1e3:.1f} us, weight-on-rows kernel {res['decode'] * 1e3:.1f} us = {gbs:.0f} GB/s of weights "
              f"({gbs / 6523.7 * 100:.0f} % of measured HBM copy bandwidth)")


def fp8_moe_decode():
    """Grouped fp8 GEMM at decode size: 32 experts of 4096 x 7168 (fc1 of a DeepSeek-V3 rank at ep 8), two tokens per
    expert, against the 128-row-tile kernel. Two weight sets are cycled (0.94 GB each: nothing stays in L2)."""
    G, N, K, per = int(os.environ.get("MFB_BENCH_EXPERTS", "32")), 4096, 7168, 2      # fewer experts for an ncu capture
    sets = []
    for _ in range(2):
        wq = torch.empty(G, N, K, dtype=torch.float8_e4m3fn, device="cuda")
        for g in range(G):
            wq[g], _ = Fn.quantize_weight_128x128(torch.randn(N, K, device="cuda") * 0.05)
        sb = torch.rand(G, N // 128, K // 128, device="cuda") * 1e-3 + 1e-4
        sets.append((wq, sb))
    T = G * 128
    xq, sa = Fn.quantize_act_1x128(bf(T, K, scale=0.7))
    bg = torch.arange(G, dtype=torch.int32, device="cuda")
    nb = torch.tensor([G], dtype=torch.int32, device="cuda")
    offs = (torch.arange(G + 1, dtype=torch.int32, device="cuda") * 128).contiguous()
    fill = torch.full((G,), per, dtype=torch.int32, device="cuda")
    res = {}
    for mode in ("tile", "decode"):
        kw = dict(block_group=bg, num_blocks=nb)
        if mode == "decode":
            kw.update(group_offsets=offs, seg_fill=fill)
        for wq, sb in sets:
            Fn.fp8_gemm(xq, sa, wq, sb, **kw)
        torch.cuda.synchronize()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        ev[0].record()
        for _ in range(3):
            for wq, sb in sets:
                Fn.fp8_gemm(xq, sa, wq, sb, **kw)
        ev[1].record()
        torch.cuda.synchronize()
        res[mode] = ev[0].elapsed_time(ev[1]) / 6
    gbs = G * N * K / res["decode"] / 1e6
    print(f"fp8 grouped decode {G} experts x {N}x{K}, {per} tokens each: 128-row tiles {res['tile'] * 1e3:.1f} us, "
          f"weight-on-rows kernel {res['decode'] * 1e3:.1f} us = {gbs:.0f} GB/s of weights "
          f"({gbs / 6523.7 * 100:.0f} % of measured HBM copy bandwidth), status {_lib.read_status()}")


def _timed(fn, iters=5, warm=2):
    for _ in range(warm):
        fn()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    torch.cuda.synchronize()
    ev[0].record()
    for _ in range(iters):
        fn()
    ev[1].record()
    torch.cuda.synchronize()
    return ev[0].elapsed_time(ev[1]) / iters


def w8a8():
    """W8A8 GEMM (int8 x int8 -> int32 in tensor memory, scales in the epilogue) at the Llama-8B linear shapes, 8192
    tokens; beside it the bf16 product of the same shape on this repository's kernel and on cuBLAS."""
    T = 8192
    for N, K, tag in ((6144, 4096, "qkv"), (4096, 4096, "proj"), (28672, 4096, "fc1"), (4096, 14336, "fc2")):
        a = torch.randint(-127, 128, (T, K), device="cuda", dtype=torch.int8)
        b = torch.randint(-127, 128, (N, K), device="cuda", dtype=torch.int8)
        sa, sb = torch.rand(T, device="cuda") * 0.01, torch.rand(N, device="cuda") * 0.01
        x, w = bf(T, K), bf(N, K, scale=0.05)
        t_i8 = _timed(lambda: Fn.w8a8_gemm(a, sa, b, sb))
        t_q = _timed(lambda: Fn.quantize_act_int8(x))
        t_bf = _timed(lambda: Fn.gemm(x, w))
        t_cb = _timed(lambda: torch.matmul(x, w.t()))
        ops = 2.0 * T * N * K
        print(f"w8a8 {tag}: T {T} N {N} K {K}: int8 {t_i8 * 1e3:.1f} us = {ops / t_i8 / 1e9:.0f} TOP/s; activation quantiser "
              f"{t_q * 1e3:.1f} us; bf16 this repository {t_bf * 1e3:.1f} us = {ops / t_bf / 1e9:.0f} TFLOP/s; cuBLAS bf16 "
              f"{t_cb * 1e3:.1f} us")


def paged_int8():
    """Paged decode attention over the int8 KV cache against the bf16 cache (same shapes as ``paged``)."""
    lib = _lib.get_lib()
    B, ctx, blk, nq, nkv, hd = 64, 2048, 128, 32, 8, 128
    nblocks = B * ctx // blk
    q = bf(B, nq, hd)
    out = torch.empty_like(q)
    tables = torch.arange(nblocks, device="cuda", dtype=torch.int32).view(B, ctx // blk).contiguous()
    lens = torch.full((B,), ctx, device="cuda", dtype=torch.int32)
    splits = lib.mfb_paged_decode_splits(B, nkv, blk, ctx // blk)
    scratch = torch.empty(lib.mfb_paged_decode_scratch_bytes(B, nq, hd, splits) // 4, device="cuda")
    for kind in ("bf16", "int8"):
        if kind == "bf16":
            kc, vc, ks, vs = bf(nblocks, blk, nkv, hd), bf(nblocks, blk, nkv, hd), None, None
            kv_bytes = 2 * B * ctx * nkv * hd * 2
        else:
            kc = torch.randint(-127, 128, (nblocks, blk, nkv, hd), device="cuda", dtype=torch.int8)
            vc = torch.randint(-127, 128, (nblocks, blk, nkv, hd), device="cuda", dtype=torch.int8)
            ks = torch.rand(nblocks, blk, nkv, device="cuda") * 0.01
            vs = torch.rand(nblocks, blk, nkv, device="cuda") * 0.01
            kv_bytes = 2 * B * ctx * nkv * (hd + 4)

        def call():
            rc = lib.mfb_paged_decode_attention_ex(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), _lib.ptr(ks), _lib.ptr(vs),
                                                   tables.data_ptr(), lens.data_ptr(), out.data_ptr(), scratch.data_ptr(),
                                                   splits, B, nq, nkv, hd, blk, ctx // blk, hd ** -0.5, _lib.stream_ptr())
            _lib.check(rc, "paged")
        ms = _timed(call, iters=5)
        print(f"paged decode, {kind} cache: {ms * 1e3:.1f} us, {kv_bytes / ms / 1e6:.0f} GB/s of cache "
              f"({kv_bytes / ms / 1e6 / 6523.7 * 100:.0f} % of measured HBM copy bandwidth)")


def bf16_decode():
    """bf16 product with a few rows of activations (decode) at the Llama-3.1-8B linear shapes: the weight-on-rows
    kernel against the general tcgen05 kernels and cuBLAS, with the weight bytes per second that each reaches. The
    weights of the shapes together (1.3 GB) exceed L2, and the calls rotate over them, so every call reads HBM."""
    shapes = ((6144, 4096, "qkv"), (4096, 4096, "proj"), (28672, 4096, "fc1"), (4096, 14336, "fc2"), (128256, 4096, "head"))
    ws = {tag: bf(N, K, scale=0.05) for N, K, tag in shapes}
    flush = torch.empty(256 * 1024 * 1024, device="cuda", dtype=torch.uint8)

    def timed_cold(fn, iters=6):
        fn()
        tot = 0.0
        for _ in range(iters):
            flush.zero_()                                  # evict the weight from L2
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            ev[0].record()
            fn()
            ev[1].record()
            torch.cuda.synchronize()
            tot += ev[0].elapsed_time(ev[1])
        return tot / iters
    for T in (1, 8, 32, 64):
        for N, K, tag in shapes:
            x, w = bf(T, K), ws[tag]
            res = {}
            for name, ks in (("auto", 0), ("ks1", 1), ("ks2", 2), ("ks4", 4), ("ks8", 8), ("occ2", 16)):
                if ks == 8 and T <= 16:
                    continue
                Fn.set_decode_gemm(True, ks)
                res[name] = timed_cold(lambda: Fn.gemm(x, w))
            Fn.set_decode_gemm(False)
            res["general"] = timed_cold(lambda: Fn.gemm(x, w))
            Fn.set_decode_gemm(True, 0)
            res["cublas"] = timed_cold(lambda: torch.matmul(x, w.t()))
            gbs = N * K * 2 / res["auto"] / 1e6
            print(f"T={T:3d} {tag:5s} N={N:6d} K={K:5d}: " + "  ".join(f"{k} {v * 1e3:7.1f} us" for k, v in res.items())
                  + f"   auto: {gbs:6.0f} GB/s = {gbs / 6523.7 * 100:.0f} % of measured HBM copy bandwidth")


def bf16_decode_one():
    """Three launches of the weight-on-rows product on one shape (8 tokens x the 28672 x 4096 up-projection, 235 MB of
    weights: larger than L2), for a profiler capture."""
    x, w = bf(8, 4096), bf(28672, 4096, scale=0.05)
    for _ in range(3):
        Fn.gemm(x, w)


def paged_tc():
    """Decode attention over the paged bf16 cache: tensor-core kernel against the CUDA-core split-KV kernel, 64 sequences
    x 2048 cached tokens (0.54 GB of K/V, larger than L2) and a short-context case (8 x 640)."""
    lib = _lib.get_lib()
    for B, ctx, blk, nq, nkv in ((64, 2048, 128, 32, 8), (64, 2048, 16, 32, 8), (8, 640, 128, 32, 8), (16, 8192, 128, 32, 8)):
        hd = 128
        per = (ctx + blk - 1) // blk
        nblocks = B * per
        q = bf(B, nq, hd)
        out = torch.empty_like(q)
        kc, vc = bf(nblocks, blk, nkv, hd), bf(nblocks, blk, nkv, hd)
        tables = torch.randperm(nblocks, device="cuda").to(torch.int32).view(B, per).contiguous()
        lens = torch.full((B,), ctx, device="cuda", dtype=torch.int32)
        kv_bytes = 2 * B * ctx * nkv * hd * 2
        s_tc = lib.mfb_paged_decode_tc_splits(B, nkv, per * blk)
        s_cc = lib.mfb_paged_decode_splits(B, nkv, blk, per)
        scratch = torch.empty(lib.mfb_paged_decode_scratch_bytes(B, nq, hd, max(s_tc, s_cc)) // 4, device="cuda")

        def tc():
            rc = lib.mfb_paged_decode_attention_tc(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), tables.data_ptr(), lens.data_ptr(),
                                                   out.data_ptr(), scratch.data_ptr(), s_tc, B, nq, nkv, nblocks, blk, per,
                                                   hd ** -0.5, _lib.status_word(q.device).data_ptr(), _lib.stream_ptr())
            _lib.check(rc, "paged tc")

        def cc():
            rc = lib.mfb_paged_decode_attention(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), tables.data_ptr(), lens.data_ptr(),
                                                out.data_ptr(), scratch.data_ptr(), s_cc, B, nq, nkv, hd, blk, per,
                                                hd ** -0.5, _lib.stream_ptr())
            _lib.check(rc, "paged")
        for name, fn, sp in (("tensor cores", tc, s_tc), ("CUDA cores", cc, s_cc)):
            ms = _timed(fn, iters=5)
            print(f"B={B} ctx={ctx} block={blk}: {name:12s} splits {sp:2d}: {ms * 1e3:7.1f} us, {kv_bytes / ms / 1e6:6.0f} GB/s of "
                  f"cache ({kv_bytes / ms / 1e6 / 6523.7 * 100:.0f} % of measured HBM copy bandwidth)")


def paged_tc_one():
    """Three launches of the tensor-core paged decode kernel (64 x 2048 tokens, block 128), for a profiler capture."""
    lib = _lib.get_lib()
    B, ctx, blk, nq, nkv, hd = 64, 2048, 128, 32, 8, 128
    per = ctx // blk
    q, out = bf(B, nq, hd), torch.empty(B, nq, hd, device="cuda", dtype=torch.bfloat16)
    kc, vc = bf(B * per, blk, nkv, hd), bf(B * per, blk, nkv, hd)
    tables = torch.arange(B * per, device="cuda", dtype=torch.int32).view(B, per).contiguous()
    lens = torch.full((B,), ctx, device="cuda", dtype=torch.int32)
    sp = lib.mfb_paged_decode_tc_splits(B, nkv, ctx)
    scratch = torch.empty(lib.mfb_paged_decode_scratch_bytes(B, nq, hd, sp) // 4, device="cuda")
    for _ in range(3):
        rc = lib.mfb_paged_decode_attention_tc(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), tables.data_ptr(), lens.data_ptr(),
                                               out.data_ptr(), scratch.data_ptr(), sp, B, nq, nkv, B * per, blk, per,
                                               hd ** -0.5, _lib.status_word(q.device).data_ptr(), _lib.stream_ptr())
        _lib.check(rc, "paged tc")


CASES = dict(paged_tc=paged_tc, paged_tc_one=paged_tc_one, bf16_decode=bf16_decode, bf16_decode_one=bf16_decode_one, w8a8=w8a8, paged_int8=paged_int8, fp8=fp8, fp8_decode=fp8_decode, fp8_moe_decode=fp8_moe_decode, gemm=gemm, grouped=grouped, fa=fa, rmsnorm=rmsnorm, swiglu=swiglu, rope=rope, ce=ce, adamw=adamw, router=router, paged=paged, mla=mla, moe=moe)

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", required=True, choices=sorted(CASES))
    a = ap.parse_args()
    torch.manual_seed(0)
    CASES[a.kernel]()
    torch.cuda.synchronize()
    print("done", a.kernel, "status", _lib.read_status())
