"""Worker (torchrun, one rank per GPU): checks the fused all-gather→GEMM and GEMM→reduce-scatter kernels
against NCCL collectives + fp32 matmul, forward and backward, and times both paths with CUDA events.
Writes a JSON summary from rank 0 to --out. NVLS is not used (plain peer loads/stores)."""
import argparse
import ctypes
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mindformers_b200.ops import _lib  # noqa: E402
from mindformers_b200.parallel import fused_tp, mappings as M, parallel_state as ps  # noqa: E402
from mindformers_b200.ops import functional as Fn  # noqa: E402


def rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def timeit(fn, iters=10):
    for _ in range(3):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def timeit_queued(fn, iters=50):
    """Device time per call with the launches queued behind a spin kernel, so that host-side launch cost does not
    show: what the call costs inside a step whose host runs ahead of the GPU."""
    for _ in range(3):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda._sleep(40_000_000)          # about 20 ms: the host enqueues all calls meanwhile
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    ap.add_argument("--T", type=int, default=4096)
    ap.add_argument("--bench", type=int, default=1)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    ps.initialize_model_parallel(tensor_model_parallel_size=world)
    tp = world
    grp = ps.get_tensor_model_parallel_group()
    res = {"tp": tp}
    T = args.T
    for (K, N, tag) in [(1024, 768, "small"), (4096, 6144 // tp * 2, "qkv"), (4096, 14336 * 2 // tp, "fc1")]:
        torch.manual_seed(5)
        x_full = (torch.randn(T, K, device="cuda") * 0.5).to(torch.bfloat16)
        w_full = (torch.randn(N * tp, K, device="cuda") * 0.05).to(torch.bfloat16)
        x_local = x_full.chunk(tp, 0)[rank].contiguous().requires_grad_()
        w = w_full.chunk(tp, 0)[rank].contiguous().requires_grad_()
        y = fused_tp.allgather_linear(x_local, w)
        g = (torch.randn(T, N, device="cuda") * 0.1).to(torch.bfloat16)
        y.backward(g)
        torch.cuda.synchronize()
        ref_y = x_full.float() @ w.detach().float().t()
        ref_dx_partial = g.float() @ w.detach().float()
        dist.all_reduce(ref_dx_partial, group=grp)
        ref_dx = ref_dx_partial.chunk(tp, 0)[rank]
        ref_dw = g.float().t() @ x_full.float()
        res[f"ag_{tag}"] = {"y": rel(y, ref_y), "dx": rel(x_local.grad, ref_dx), "dw": rel(w.grad, ref_dw)}
    for (K, N, tag) in [(768, 1024, "small"), (4096 // tp * 2, 4096, "proj"), (14336 // tp, 4096, "fc2")]:
        torch.manual_seed(6)
        x = (torch.randn(T, K, device="cuda") * 0.5 + rank).to(torch.bfloat16).requires_grad_()
        w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
        y = fused_tp.linear_reduce_scatter(x, w)
        g_local = (torch.randn(T // tp, N, device="cuda") * 0.1 + 0.01 * rank).to(torch.bfloat16)
        y.backward(g_local)
        torch.cuda.synchronize()
        part = x.detach().float() @ w.detach().float().t()
        dist.all_reduce(part, group=grp)
        ref_y = part.chunk(tp, 0)[rank]
        g_full = M.all_gather_first_dim(g_local, grp, tp)
        ref_dx = g_full.float() @ w.detach().float()
        ref_dw = g_full.float().t() @ x.detach().float()
        res[f"rs_{tag}"] = {"y": rel(y, ref_y), "dx": rel(x.grad, ref_dx), "dw": rel(w.grad, ref_dw)}
    # GEMM -> all-reduce (inference): any token count, identical bits on every rank
    for (Tq, K, N, tag) in [(1, 1024, 512, "decode1"), (64, 7168 // tp, 2048, "decode64"), (200, 768, 1024, "odd"),
                            (2048, 14336 // tp, 4096, "prefill")]:
        torch.manual_seed(8)
        x = (torch.randn(Tq, K, device="cuda") * 0.5 + 0.1 * rank).to(torch.bfloat16)
        w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
        y = fused_tp.gemm_all_reduce(x, w)
        y2 = fused_tp.gemm_all_reduce(x, w)          # the next call lands in the other parity
        part = x.float() @ w.float().t()
        dist.all_reduce(part, group=grp)
        same = [torch.empty_like(y) for _ in range(tp)]
        dist.all_gather(same, y, group=grp)
        res[f"ar_{tag}"] = {"y": rel(y, part), "repeat": rel(y2, part),
                            "rank_mismatch": float(max((s - same[0]).abs().max().item() for s in same))}
    res["status"] = _lib.read_status()
    if args.bench:
        for (Tq, K3, N3, tag) in [(64, 14336 // tp, 4096, "decode64_fc2"), (1024, 14336 // tp, 4096, "chunk1024_fc2")]:
            x3 = torch.randn(Tq, K3, device="cuda").to(torch.bfloat16)
            w3 = (torch.randn(N3, K3, device="cuda") * 0.05).to(torch.bfloat16)
            t_f = timeit(lambda: fused_tp.gemm_all_reduce(x3, w3), iters=50)
            t_n = timeit(lambda: M.all_reduce(torch.matmul(x3, w3.t()), grp, tp), iters=50)
            res[f"bench_ar_{tag}"] = {"fused_ms": t_f, "nccl_cublas_ms": t_n,
                                      "fused_queued_ms": timeit_queued(lambda: fused_tp.gemm_all_reduce(x3, w3)),
                                      "nccl_cublas_queued_ms": timeit_queued(
                                          lambda: M.all_reduce(torch.matmul(x3, w3.t()), grp, tp)),
                                      "bytes_over_nvlink": (tp - 1) * Tq * N3 * 2,
                                      "nvlink_floor_ms": (tp - 1) * Tq * N3 * 2 / 770e9 * 1e3,
                                      "gemm_floor_ms": 2.0 * Tq * N3 * K3 / 1415.7e12 * 1e3,
                                      "weight_read_floor_ms": N3 * K3 * 2 / 6523.7e9 * 1e3}
        K, N = 4096, 14336 * 2 // tp
        x_local = (torch.randn(T // tp, K, device="cuda")).to(torch.bfloat16)
        w = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
        t_f = timeit(lambda: fused_tp.allgather_gemm(x_local, w))
        t_n = timeit(lambda: torch.matmul(M.all_gather_first_dim(x_local, grp, tp), w.t()))
        t_g = timeit(lambda: Fn.gemm(torch.empty(T, K, device="cuda", dtype=torch.bfloat16), w))
        fl = 2.0 * T * N * K
        res["bench_ag_fc1"] = {"fused_ms": t_f, "nccl_cublas_ms": t_n, "gemm_only_ms": t_g,
                               "fused_tflops": fl / t_f / 1e9, "bytes_over_nvlink": (T - T // tp) * K * 2,
                               "nvlink_floor_ms": (T - T // tp) * K * 2 / 770e9 * 1e3}
        K2, N2 = 14336 // tp, 4096
        x2 = (torch.randn(T, K2, device="cuda")).to(torch.bfloat16)
        w2 = (torch.randn(N2, K2, device="cuda") * 0.05).to(torch.bfloat16)
        t_f = timeit(lambda: fused_tp.gemm_reduce_scatter(x2, w2))
        t_n = timeit(lambda: M.reduce_scatter_first_dim(torch.matmul(x2, w2.t()), grp, tp))
        t_g = timeit(lambda: Fn.gemm(x2, w2))
        fl = 2.0 * T * N2 * K2
        res["bench_rs_fc2"] = {"fused_ms": t_f, "nccl_cublas_ms": t_n, "gemm_only_ms": t_g,
                               "fused_tflops": fl / t_f / 1e9, "bytes_over_nvlink": (T - T // tp) * N2 * 2,
                               "nvlink_floor_ms": (T - T // tp) * N2 * 2 / 770e9 * 1e3}
        # short reduction dimensions (attention output projection, dgrad of the QKV projection): the link-bound cases
        lib = _lib.get_lib()
        for tag, K4, N4, bmn in (("rs_proj", 4096 // tp, 4096, False), ("rs_qkv_dgrad", 6144 // tp, 4096, True)):
            x4 = torch.randn(T, K4, device="cuda").to(torch.bfloat16)
            w4 = (torch.randn((K4, N4) if bmn else (N4, K4), device="cuda") * 0.05).to(torch.bfloat16)
            row = {}
            for mode in (0, 1):
                lib.mfb_tp_set_rs_interleave(mode)
                row["interleaved_ms" if mode else "chunk_order_ms"] = timeit(lambda: fused_tp.gemm_reduce_scatter(x4, w4, b_mn=bmn))
            if hasattr(lib, "mfb_tp_set_probe"):
                lib.mfb_tp_set_probe.argtypes = [ctypes.c_int]
                lib.mfb_tp_set_probe.restype = None
                for bits, name in ((1, "probe_no_peer_stores_ms"), (2, "probe_no_partial_reads_ms"), (3, "probe_neither_ms")):
                    lib.mfb_tp_set_probe(bits)
                    row[name] = timeit(lambda: fused_tp.gemm_reduce_scatter(x4, w4, b_mn=bmn))
                lib.mfb_tp_set_probe(0)
            row["nccl_cublas_ms"] = timeit(lambda: M.reduce_scatter_first_dim(torch.matmul(x4, w4 if bmn else w4.t()), grp, tp))
            row["gemm_only_ms"] = timeit(lambda: Fn.gemm(x4, w4, b_mn=bmn))
            res[f"bench_{tag}"] = row
        # all-gather -> GEMM where the GEMM is short against the transfer: the QKV projection and the two input-gradient
        # GEMMs behind a row-parallel layer (gathered output gradient times the weight)
        for tag, K5, N5, bmn in (("ag_qkv", 4096, 6144 // tp, False), ("ag_proj_dgrad", 4096, 4096 // tp, True),
                                 ("ag_fc2_dgrad", 4096, 14336 // tp, True)):
            x5 = torch.randn(T // tp, K5, device="cuda").to(torch.bfloat16)
            w5 = (torch.randn((K5, N5) if bmn else (N5, K5), device="cuda") * 0.05).to(torch.bfloat16)
            x5_full = torch.empty(T, K5, device="cuda", dtype=torch.bfloat16)
            res[f"bench_{tag}"] = {
                "fused_ms": timeit(lambda: fused_tp.allgather_gemm(x5, w5, b_mn=bmn)),
                "nccl_cublas_ms": timeit(lambda: torch.matmul(M.all_gather_first_dim(x5, grp, tp), w5 if bmn else w5.t())),
                "gemm_only_ms": timeit(lambda: Fn.gemm(x5_full, w5, b_mn=bmn)),
                "bytes_over_nvlink": (T - T // tp) * K5 * 2, "nvlink_floor_ms": (T - T // tp) * K5 * 2 / 770e9 * 1e3}
        lib.mfb_tp_set_rs_interleave(0)
        res["bench_rs_fc2"]["chunk_order_ms"] = timeit(lambda: fused_tp.gemm_reduce_scatter(x2, w2))
        lib.mfb_tp_set_rs_interleave(1)
        res["status_after_bench"] = _lib.read_status()
    if rank == 0:
        print(json.dumps(res, indent=1))
        if args.out:
            with open(args.out, "w") as f:
                json.dump(res, f, indent=1)
    worst = max(v for key, d in res.items() if isinstance(d, dict) and not key.startswith("bench") for v in d.values())
    ok = worst < 1e-2 and res.get("status", 0) == 0
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
