"""Worker (torchrun, one rank per GPU): the MoE layer through the device-side exchange kernels against the NCCL
all-to-all-v dispatcher on the same weights and tokens (expert parallel = world size), forward and backward, then a
timing of a Qwen3-30B-A3B-shaped layer both ways. Writes a JSON summary from rank 0 to --out."""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mindformers_b200.ops import _lib  # noqa: E402
from mindformers_b200.parallel import parallel_state as ps  # noqa: E402
from mindformers_b200.parallel.layers.moe import MoELayer  # noqa: E402
from mindformers_b200.parallel.transformer_config import TransformerConfig  # noqa: E402


def make(H, E, k, F, ep):
    cfg = TransformerConfig(num_layers=1, hidden_size=H, num_attention_heads=4, ffn_hidden_size=4 * H, num_moe_experts=E,
                            moe_router_topk=k, moe_ffn_hidden_size=F, params_dtype=torch.bfloat16, compute_dtype=torch.bfloat16,
                            moe_aux_loss_coeff=1e-2, expert_model_parallel_size=ep)
    cfg.device = "cuda"
    torch.manual_seed(7)
    return cfg, MoELayer(cfg).train()


def run(layer, cfg, x, fused):
    cfg.fused_moe_comm = fused
    xi = x.clone().requires_grad_()
    for p in layer.parameters():
        p.grad = None
    y, aux = layer(xi)
    (y.float().pow(2).mean() + aux).backward()
    return [y.detach().float(), xi.grad.float(), layer.router.weight.grad.float().clone(),
            layer.experts.weight1.grad.float().clone(), layer.experts.weight2.grad.float().clone()]


def timeit(fn, iters=8):
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    ap.add_argument("--bench", type=int, default=1)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    ps.initialize_model_parallel(tensor_model_parallel_size=1, expert_model_parallel_size=world)
    res = {"ep": world}
    cfg, layer = make(256, 8 * world, 2, 128, world)
    g = torch.Generator(device="cuda").manual_seed(50 + rank)
    x = (torch.randn(1000 + 24 * rank, 256, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    a = run(layer, cfg, x, True)
    b = run(layer, cfg, x, False)
    names = ["y", "dx", "d_router", "d_w1", "d_w2"]
    errs = {n: ((p - q).norm() / (q.norm() + 1e-12)).item() for n, p, q in zip(names, a, b)}
    res["rel_err_vs_nccl"] = errs
    res["status"] = _lib.read_status()
    # receive buffers that are too small: the plan kernel reports the overflow, adapt_capacity grows the buffers on
    # all ranks together, and the layer then matches the NCCL path again
    from mindformers_b200.parallel import fused_moe
    ex = fused_moe.MoEExchange.get(cfg)
    ex.factor = 0.3
    ex._shared.clear()
    grown = 0
    for _ in range(8):
        a2 = run(layer, cfg, x, True)
        if not fused_moe.adapt_capacity():
            break
        grown += 1
    res["capacity_growth_steps"] = grown
    res["capacity_factor"] = ex.factor
    res["rel_err_after_growth"] = max(((p - q).norm() / (q.norm() + 1e-12)).item() for p, q in zip(a2, b))
    res["status_after_growth"] = _lib.read_status()
    if args.bench:
        cfg2, big = make(2048, 128, 8, 768, world)
        T = 4096
        xb = (torch.randn(T, 2048, device="cuda") * 0.5).to(torch.bfloat16)
        t_f = timeit(lambda: run(big, cfg2, xb, True))
        t_n = timeit(lambda: run(big, cfg2, xb, False))
        copies = T * 8
        remote = copies * (world - 1) / world * 2048 * 2          # bytes this rank sends (and receives) per exchange
        flops = 3 * 2 * copies * 2048 * 768 * 3                   # fwd + dgrad + wgrad of the two grouped GEMMs
        res["bench_qwen3_30b_layer"] = {
            "T": T, "fused_fwd_bwd_ms": t_f, "nccl_fwd_bwd_ms": t_n, "exchanges": 4, "remote_bytes_per_exchange": remote,
            "nvlink_floor_ms": 4 * remote / 770e9 * 1e3, "gemm_floor_ms": flops / 1415.7e12 * 1e3}
        res["status_after_bench"] = _lib.read_status()
    if rank == 0:
        print(json.dumps(res, indent=1))
        if args.out:
            with open(args.out, "w") as f:
                json.dump(res, f, indent=1)
    ok = (res["status"] == 0 and max(errs.values()) < 3e-2 and res["capacity_growth_steps"] >= 1
          and res["rel_err_after_growth"] < 3e-2 and res["status_after_growth"] == 0)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
