"""Worker (torchrun, one rank per GPU): the low-latency all-reduce against the fp32 sum of the gathered inputs and
against NCCL's timing. Covers: sizes from one vector to the buffer limit, changing sizes between consecutive calls (the
reset of older generations), inputs that contain negative zeros, in-place output, bit equality across ranks, and a
CUDA-graph capture replayed with new inputs. Writes a JSON summary from rank 0 to --out."""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mindformers_b200.ops import _lib  # noqa: E402
from mindformers_b200.parallel import ll_allreduce  # noqa: E402


def reference(x, world):
    parts = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(parts, x)
    acc = torch.zeros_like(x, dtype=torch.float32)
    for p in parts:                     # rank order, fp32: the kernel's order
        acc += p.float()
    return acc.to(torch.bfloat16)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    group = dist.group.WORLD
    ar = ll_allreduce.get(group)
    res = {"world": world, "max_bytes": ar.max_bytes}
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    worst, mismatch_between_ranks, calls = 0.0, 0.0, 0
    sizes = [8, 4096, 8 * 7168, 64 * 7168, 24, 64 * 7168, 8, ar.max_bytes // 2, 1000 * 8, 16 * 7168, 64 * 7168, 8]
    for n in sizes:
        x = torch.randn(n, device="cuda", generator=g).to(torch.bfloat16)
        x[::5] = 0.0
        x[1::7] = -0.0                  # the sentinel value as data
        ref = reference(x, world)
        y = ar(x)
        torch.cuda.synchronize()
        worst = max(worst, (y.float() - ref.float()).abs().max().item())
        other = y.clone()
        dist.broadcast(other, src=0)
        mismatch_between_ranks = max(mismatch_between_ranks, (other.float() - y.float()).abs().max().item())
        z = x.clone()
        ar(z, out=z)                    # in place
        torch.cuda.synchronize()
        worst = max(worst, (z.float() - ref.float()).abs().max().item())
        calls += 2
    res.update(max_abs_diff_vs_fp32_sum=worst, max_diff_between_ranks=mismatch_between_ranks, calls=calls)
    # CUDA graph: capture one call, replay with new inputs
    n = 64 * 7168
    static_in = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    static_out = torch.empty_like(static_in)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        ar(static_in, out=static_out)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    dist.barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ar(static_in, out=static_out)
    graph_worst = 0.0
    for it in range(7):
        x = torch.randn(n, device="cuda", generator=g).to(torch.bfloat16)
        ref = reference(x, world)
        static_in.copy_(x)
        graph.replay()
        torch.cuda.synchronize()
        graph_worst = max(graph_worst, (static_out.float() - ref.float()).abs().max().item())
    res["graph_replay_max_abs_diff"] = graph_worst
    # timing against NCCL (device time of 20 back-to-back calls, max over ranks)
    timing = {}
    for tokens in (1, 8, 64, 128):
        n = tokens * 7168
        if n * 2 > ar.max_bytes:
            continue
        x = torch.randn(n, device="cuda", generator=g).to(torch.bfloat16)
        y = torch.empty_like(x)
        row = {}
        for name, fn in (("ll", lambda: ar(x, out=y)), ("nccl", lambda: dist.all_reduce(y))):
            for _ in range(5):
                fn()
            dist.barrier()
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(20):
                fn()
            e.record()
            torch.cuda.synchronize()
            t = torch.tensor([s.elapsed_time(e) / 20 * 1e3], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            row[name + "_us"] = round(t.item(), 2)
        timing[f"{tokens}x7168"] = row
    res["timing"] = timing
    res["status"] = _lib.read_status()
    if rank == 0:
        print(json.dumps(res, indent=1))
        if args.out:
            with open(args.out, "w") as f:
                json.dump(res, f, indent=1)
    ok = res["status"] == 0 and worst == 0.0 and mismatch_between_ranks == 0.0 and graph_worst == 0.0
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
