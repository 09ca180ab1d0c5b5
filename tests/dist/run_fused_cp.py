"""Worker (torchrun, one rank per GPU): context-parallel attention through the peer-memory K/V exchange + rectangular
flash attention against full-sequence fp32 attention, forward and backward, contiguous and zig-zag layouts; then a
timing against the NCCL all-gather path at a long-context shape. Writes a JSON summary from rank 0 to --out."""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mindformers_b200.ops import _lib  # noqa: E402
from mindformers_b200.ops import functional as Fn  # noqa: E402
from mindformers_b200.parallel import fused_cp, parallel_state as ps  # noqa: E402


def rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    ap.add_argument("--bench", type=int, default=1)
    ap.add_argument("--bench-seq", type=int, default=16384, help="tokens per rank of the timing case")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    ps.initialize_model_parallel(context_parallel_size=world)
    res = {"cp": world}
    nq, nkv, S = 8, 2, 512
    St = S * world
    worst = 0.0
    for zigzag in (False, True):
        torch.manual_seed(3)
        qf = (torch.randn(1, St, nq, 128, device="cuda") * 0.5).to(torch.bfloat16)
        kf = (torch.randn(1, St, nkv, 128, device="cuda") * 0.5).to(torch.bfloat16)
        vf = (torch.randn(1, St, nkv, 128, device="cuda") * 0.5).to(torch.bfloat16)
        gf = (torch.randn(1, St, nq, 128, device="cuda") * 0.1).to(torch.bfloat16)
        cut = (lambda t: fused_cp.zigzag_slice(t, world, rank)) if zigzag else (lambda t: t.chunk(world, dim=1)[rank])
        q, k, v = (cut(t).contiguous().requires_grad_() for t in (qf, kf, vf))
        o = fused_cp.fused_cp_attention(q, k, v, 128 ** -0.5, zigzag)
        o.backward(cut(gf).contiguous())
        qr, kr, vr = (t.float().requires_grad_() for t in (qf, kf, vf))
        ref = Fn.attention_reference(qr, kr, vr, True, 128 ** -0.5)
        ref.backward(gf.float())
        errs = {"o": rel(o, cut(ref)), "dq": rel(q.grad, cut(qr.grad)), "dk": rel(k.grad, cut(kr.grad)),
                "dv": rel(v.grad, cut(vr.grad))}
        res["zigzag" if zigzag else "contiguous"] = errs
        worst = max(worst, max(errs.values()))
        # the ring: K/V blocks over NCCL send / recv under the flash kernels of the block at hand, memory O(S / cp)
        from mindformers_b200.parallel.ring_attention import ring_attention
        q2, k2, v2 = (cut(t).contiguous().requires_grad_() for t in (qf, kf, vf))
        o2 = ring_attention(q2, k2, v2, 128 ** -0.5, zigzag=zigzag)
        o2.backward(cut(gf).contiguous())
        errs2 = {"o": rel(o2, cut(ref)), "dq": rel(q2.grad, cut(qr.grad)), "dk": rel(k2.grad, cut(kr.grad)),
                 "dv": rel(v2.grad, cut(vr.grad))}
        res["ring_zigzag" if zigzag else "ring_contiguous"] = errs2
        worst = max(worst, max(errs2.values()))
    res["status"] = _lib.read_status()
    if args.bench:
        S, nq, nkv = args.bench_seq, 28, 4        # Qwen2.5-7B heads; S tokens per rank
        q = (torch.randn(1, S, nq, 128, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
        k = (torch.randn(1, S, nkv, 128, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
        v = (torch.randn(1, S, nkv, 128, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
        g = (torch.randn(1, S, nq, 128, device="cuda") * 0.1).to(torch.bfloat16)

        def run(zz):
            o = fused_cp.fused_cp_attention(q, k, v, 128 ** -0.5, zz)
            o.backward(g)

        def timeit(fn, iters=5):
            for _ in range(2):
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
        St = S * world
        flops_total = 4 * St * St / 2 * 128 * nq * 3.5       # fwd + bwd (2.5x) causal, whole sequence
        kv_bytes = 2 * S * nkv * 128 * 2 * (world - 1)        # inbound K,V per gather (two gathers + one reduce-scatter)
        t_c, t_z = timeit(lambda: run(False)), timeit(lambda: run(True))
        from mindformers_b200.parallel.ring_attention import ring_attention

        def run_ring(zz):
            o = ring_attention(q, k, v, 128 ** -0.5, zigzag=zz)
            o.backward(g)
        t_rc, t_rz = timeit(lambda: run_ring(False)), timeit(lambda: run_ring(True))
        res["bench"] = {"tokens_per_rank": S, "contiguous_ms": t_c, "zigzag_ms": t_z,
                        "ring_contiguous_ms": t_rc, "ring_zigzag_ms": t_rz,
                        "attn_floor_ms_per_rank": flops_total / world / 1415.7e12 * 1e3,
                        "nvlink_floor_ms": 3 * kv_bytes / 770e9 * 1e3,
                        "zigzag_tflops_per_rank": flops_total / world / t_z / 1e9}
        res["status_after_bench"] = _lib.read_status()
    if rank == 0:
        print(json.dumps(res, indent=1))
        if args.out:
            with open(args.out, "w") as f:
                json.dump(res, f, indent=1)
    ok = res["status"] == 0 and worst < 3e-2
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
