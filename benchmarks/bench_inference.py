"""Offline generation benchmark on random-init weights: batch of random prompts, greedy decode.

One rank per GPU under ``torch.distributed.run``; tensor-parallel attention over all ranks, experts expert-parallel
over the same ranks (``--ep``), optional block-scaled fp8 weights (``--fp8``), paged KV cache with ``--block`` tokens
per block. Reports, as one JSON line from rank 0: time to first token of the batch (prefill, device-timed), decode
tokens/s over the whole batch (generated tokens / decode time, device-timed, max over ranks) and the end-to-end
tokens/s the reference quotes (generated tokens / total wall time, ``generation/text_generator.py:1108-1111``).

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/bench_inference.py \\
        --preset deepseek_v3 --layers 8 --ep 8 --fp8 --batch 64 --prompt 2048 --new 256 --block 128
"""
import argparse
import json
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="deepseek_v3")
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--ep", type=int, default=None, help="expert-parallel size (default: world size for MoE presets)")
    ap.add_argument("--fp8", action="store_true")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--new", type=int, default=256)
    ap.add_argument("--block", type=int, default=128)
    ap.add_argument("--graph", action="store_true", help="capture the decode step in a CUDA graph")
    ap.add_argument("--hidden", type=int, default=None, help="debug only: override the hidden size")
    ap.add_argument("--experts", type=int, default=None, help="debug only: override the number of routed experts")
    args = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    from mindformers_b200.inference.fp8 import quantize_model_fp8
    from mindformers_b200.models import AutoModel
    from mindformers_b200.models.presets import get_preset
    from mindformers_b200.ops import _lib
    from mindformers_b200.parallel import parallel_state as ps

    cfg = get_preset(args.preset)
    cfg["num_hidden_layers"] = args.layers
    cfg.pop("num_nextn_predict_layers", None)            # the multi-token-prediction head is a training component
    if args.hidden:
        cfg["hidden_size"] = args.hidden
    if args.experts:
        cfg["n_routed_experts"] = args.experts
    moe = bool(cfg.get("n_routed_experts") or cfg.get("num_experts"))
    ep = (args.ep or world) if moe else 1
    ps.initialize_model_parallel(tensor_model_parallel_size=world, expert_model_parallel_size=ep,
                                 expert_tensor_parallel_size=1 if ep > 1 else None)
    torch.manual_seed(1234)
    extra = dict(tensor_model_parallel_size=world, block_size=args.block, seq_length=args.prompt + args.new,
                 max_position_embeddings=max(args.prompt + args.new, 4096), fused_tp_comm=True)
    if ep > 1:
        extra.update(expert_model_parallel_size=ep, expert_tensor_parallel_size=1)
    model = AutoModel.from_config(cfg, device="cuda", **extra).eval()
    fp8_stats = quantize_model_fp8(model) if args.fp8 else None
    torch.cuda.synchronize()
    mem_weights = torch.cuda.memory_allocated() / 2 ** 30

    g = torch.Generator().manual_seed(7)                 # the same prompts on every rank
    vocab = cfg["vocab_size"]
    prompts = torch.randint(3, vocab, (args.batch, args.prompt), generator=g).tolist()

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    gen_kw = dict(do_sample=False, eos_token_id=None)
    model.generate([p[:128] for p in prompts[:2]], max_new_tokens=4, **gen_kw)       # warm-up (allocations, buffers)
    model.generate(prompts, max_new_tokens=1, **gen_kw)
    sync()
    # time to first token: prefill of the whole batch + one sampling step
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    _lib.reset_launch_count()
    ev[0].record()
    model.generate(prompts, max_new_tokens=1, **gen_kw)
    ev[1].record()
    sync()
    ttft_ms = ev[0].elapsed_time(ev[1])
    t0 = time.perf_counter()
    ev[2].record()
    out = model.generate(prompts, max_new_tokens=args.new, **gen_kw)
    ev[3].record()
    sync()
    wall = time.perf_counter() - t0
    total_ms = ev[2].elapsed_time(ev[3])
    launches = _lib.launch_count()
    graph_ms = loop_ms = loop2_ms = 0.0
    if args.graph:
        # the same generation with the decode step replayed from a CUDA graph (captured inside the call: its cost is
        # part of the time): first with the token selection on the host after every step, then with the selection and
        # the state update on the device (tokens read back once per burst), whose second call reuses the capture
        def timed(**kw):
            evg = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            evg[0].record()
            res = model.generate(prompts, max_new_tokens=args.new, use_cuda_graph=True, **kw, **gen_kw)
            evg[1].record()
            sync()
            return evg[0].elapsed_time(evg[1]), res
        graph_ms, out_g = timed(device_loop=False)
        graph_same = sum(a == b for a, b in zip(out, out_g)) / len(out)
        loop_ms, out_l = timed(device_loop=True)
        loop2_ms, out_l2 = timed(device_loop=True)
        loop_same = sum(a == b for a, b in zip(out, out_l)) / len(out)
        loop_same2 = sum(a == b for a, b in zip(out, out_l2)) / len(out)
    t = torch.tensor([ttft_ms, total_ms, graph_ms, loop_ms, loop2_ms], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ttft_ms, total_ms, graph_ms, loop_ms, loop2_ms = t.tolist()
    new_tokens = sum(len(o) - args.prompt for o in out)
    decode_ms = max(total_ms - ttft_ms, 1e-6)
    if rank == 0:
        print(json.dumps({
            "metric": "decode tokens/s (batch) and time to first token", "decode_tokens_per_s": (new_tokens - args.batch) / decode_ms * 1e3,
            "ttft_ms": ttft_ms, "prefill_tokens_per_s": args.batch * args.prompt / ttft_ms * 1e3,
            "end_to_end_tokens_per_s": new_tokens / wall, "ms_per_decode_step": decode_ms / max(args.new - 1, 1),
            "n_gpus": world, "dtype": "fp8 e4m3 block-scaled weights, bf16 activations" if args.fp8 else "bf16",
            "data": "synthetic uniform token ids, random-init weights", "new_tokens": new_tokens,
            "config": {"model": f"{args.preset}(layers={args.layers})", "batch": args.batch, "prompt": args.prompt,
                       "new": args.new, "block_size": args.block, "parallelism": f"tp{world} ep{ep}"},
            "cuda_graph_decode": None if not args.graph else {
                "decode_tokens_per_s": (new_tokens - args.batch) / max(graph_ms - ttft_ms, 1e-6) * 1e3,
                "ms_per_decode_step": max(graph_ms - ttft_ms, 1e-6) / max(args.new - 1, 1),
                "sequences_equal_to_eager": graph_same},
            "device_loop_decode": None if not args.graph else {
                "decode_tokens_per_s_first_call": (new_tokens - args.batch) / max(loop_ms - ttft_ms, 1e-6) * 1e3,
                "decode_tokens_per_s": (new_tokens - args.batch) / max(loop2_ms - ttft_ms, 1e-6) * 1e3,
                "ms_per_decode_step": max(loop2_ms - ttft_ms, 1e-6) / max(args.new - 1, 1),
                "sequences_equal_to_eager": [loop_same, loop_same2]},
            "weights_gib_per_gpu": round(mem_weights, 2), "fp8": fp8_stats, "gpu_launches": launches,
            "kernel_status_word": _lib.read_status()}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
