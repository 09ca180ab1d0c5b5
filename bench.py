#!/usr/bin/env python
"""Headline benchmark: Llama-3.1-8B pre-training throughput (tokens/s, whole job) on N B200 GPUs.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Config (weak scaling, 8 sequences of 4096 tokens per GPU per step, so N=8 is the global batch of 64):
32 layers, hidden 4096, 32 heads / 8 KV heads, FFN 14336, vocab 128256, RoPE theta 5e5 (Llama-3
scaling), bf16 compute, fp32 gradient accumulation and AdamW state, tensor parallel 2 with sequence
parallelism once N >= 2, data parallel N/2 with the sharded optimizer, micro batch 1. Synthetic uniform
token ids, random-init weights.

Prints ONE JSON line on rank 0. ``value`` is device-timed (CUDA events, max over ranks, barrier and
synchronize on both sides); ``e2e`` repeats the measurement through ``TrainingEngine.train_step`` with
the host→device copy of the tokens from pinned memory and the device→host read of the loss inside the
timed region. ``--impl reference`` reports why the reference itself cannot run here.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BASELINE_TOKENS_PER_S_PER_DEVICE = 2703.0  # Llama-3.1-8B finetune, research/llama3_1/README.md:24 (Ascend 910B)


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.rows, self._halt = index, [], threading.Event()

    def run(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,power.draw")
        while not self._halt.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={q}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5)
                parts = [p.strip() for p in out.stdout.strip().split(",")]
                if len(parts) >= 7:
                    self.rows.append(parts)
            except Exception:
                pass
            self._halt.wait(0.2)

    def stop(self):
        self._halt.set()
        self.join(timeout=3)
        sm = [float(r[0]) for r in self.rows if r[0].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        mx = [float(r[1]) for r in self.rows if r[1].replace(".", "").isdigit()]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(self.rows)}


def reference_arm(args):
    why = ("reference needs MindSpore + Ascend CANN: `import mindformers` from baseline/_ref fails with "
           "ModuleNotFoundError: No module named 'mindspore' (not installable offline; no CUDA backend in the reference)")
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "baseline"])
    ap.add_argument("--seqs-per-gpu", type=int, default=8)
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--model", default="llama3_1_8b")
    ap.add_argument("--layers", type=int, default=None, help="debug only: fewer layers (result is not a valid bench)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--tp", type=int, default=None)
    ap.add_argument("--recompute", type=int, default=0, help="recompute the activations of the first N layers in backward")
    ap.add_argument("--config", default="llama8b", choices=["llama8b", "qwen3_moe", "qwen25_cp"],
                    help="llama8b: the headline (Llama-3.1-8B, TP2+SP x DP); qwen3_moe: Qwen3-30B-A3B, expert parallel = N, "
                         "micro batch 1; qwen25_cp: Qwen2.5-7B, one sequence of --seq-len tokens, context parallel = N")
    args = ap.parse_args()
    if args.config == "qwen3_moe" and args.model == "llama3_1_8b":
        args.model = "qwen3_30b_a3b"
    if args.config == "qwen25_cp" and args.model == "llama3_1_8b":
        args.model = "qwen2_5_7b"
        if args.seq_len == 4096:
            args.seq_len = 131072
        args.seqs_per_gpu = 1
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run for --gpus > 1")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    from mindformers_b200.models.presets import get_preset
    from mindformers_b200.ops import _lib
    from mindformers_b200.ops import functional as Fn
    from mindformers_b200.parallel import fused_comm, parallel_state as ps
    from mindformers_b200.trainer.engine import TrainingEngine

    if args.impl == "baseline":       # library path: cuBLAS GEMM, SDPA attention, NCCL collectives only
        Fn.set_gemm_backend("cublas")
        Fn.set_attention_backend("sdpa")
        fused_comm.set_enabled(False)

    tp = args.tp or (2 if world >= 2 else 1)
    cp = ep = 1
    if args.config == "qwen3_moe":
        tp, ep = args.tp or 1, world
    elif args.config == "qwen25_cp":
        tp, cp = args.tp or 1, world
    ps.initialize_model_parallel(tensor_model_parallel_size=tp, context_parallel_size=cp, expert_model_parallel_size=ep,
                                 expert_tensor_parallel_size=1 if ep > 1 else None)
    dp = world // (tp * cp)
    torch.manual_seed(1234)
    preset = get_preset(args.model)
    if args.layers:
        preset["num_hidden_layers"] = args.layers
    parallel = dict(tensor_model_parallel_size=tp, sequence_parallel=tp > 1)
    extra = {}
    if ep > 1:
        parallel.update(expert_model_parallel_size=ep, expert_tensor_parallel_size=1)
    if cp > 1:
        parallel.update(context_parallel_size=cp)
        extra.update(cp_comm_type="p2p", cp_zigzag=True)
    engine = TrainingEngine.from_model_config(
        preset, parallel=parallel, seq_length=args.seq_len, learning_rate=1e-4, betas=(0.9, 0.95), weight_decay=0.1,
        max_grad_norm=1.0, micro_batch_size=1,
        recompute=([args.recompute] if args.recompute else False), **extra)
    S, V = args.seq_len, preset["vocab_size"]
    n_batches = args.warmup + args.steps
    if cp > 1:
        # one sequence of S tokens over the context-parallel group, zig-zag chunks (rank r: chunks r and 2cp-1-r)
        from mindformers_b200.parallel.fused_cp import zigzag_slice
        seqs_local = args.seqs_per_gpu
        g = torch.Generator().manual_seed(100 + ps.get_data_parallel_rank())
        r = ps.get_context_parallel_rank()
        host = []
        for _ in range(2):
            full = torch.randint(0, V, (seqs_local, S + 1), generator=g, dtype=torch.int64)
            pos = torch.arange(S).unsqueeze(0).expand(seqs_local, S)
            host.append({"input_ids": zigzag_slice(full[:, :-1], cp, r).contiguous().pin_memory(),
                         "labels": zigzag_slice(full[:, 1:], cp, r).contiguous().pin_memory(),
                         "position_ids": zigzag_slice(pos, cp, r).contiguous().pin_memory()})

        def host_batch(i):
            return host[i % 2]
    else:
        seqs_local = args.seqs_per_gpu * world // dp          # sequences this data-parallel rank handles per step
        g = torch.Generator().manual_seed(100 + ps.get_data_parallel_rank())
        host = [torch.randint(0, V, (seqs_local, S + 1), generator=g, dtype=torch.int64).pin_memory() for _ in range(2)]

        def host_batch(i):
            t = host[i % 2]
            return {"input_ids": t[:, :-1], "labels": t[:, 1:]}

    dev_batches = [{k: v.cuda().contiguous() for k, v in host_batch(i).items()} for i in range(2)]

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        sync()
        sampler = ClockSampler(local_rank)
        sampler.start()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        _lib.reset_launch_count()
        start.record()
        last = None
        for i in range(steps):
            last = fn(i)
        end.record()
        sync()
        clocks = sampler.stop()
        ms = start.elapsed_time(end)
        t = torch.tensor([ms], device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item(), clocks, _lib.launch_count(), last

    # ---- device-timed metric ---------------------------------------------------------------------
    for i in range(args.warmup):
        out = engine.train_step_device(dev_batches[i % 2])
        engine.adapt_moe_capacity()     # expert-parallel receive buffers grow here if routing overflowed them
    total_ms, clocks, launches, out = timed(lambda i: engine.train_step_device(dev_batches[i % 2]), args.steps)
    loss_val = float(out["loss"])
    tokens_per_step = (args.seqs_per_gpu * S) if cp > 1 else args.seqs_per_gpu * world * S
    ms_per_step = total_ms / args.steps
    value = tokens_per_step / (ms_per_step / 1e3)

    # ---- end to end through the public API ---------------------------------------------------------
    e2e = None
    if not args.no_e2e:
        engine.train_step(host_batch(0))
        e2e_ms, _, _, _ = timed(lambda i: engine.train_step(host_batch(i)), args.steps)
        e2e = {"value": tokens_per_step / (e2e_ms / args.steps / 1e3), "unit": "tokens/s",
               "h2d_bytes_per_step": engine.h2d_bytes, "d2h_bytes_per_step": engine.d2h_bytes,
               "api": "mindformers_b200.trainer.engine.TrainingEngine.train_step"}

    status = _lib.read_status()
    if rank == 0:
        line = {
            "metric": "train tokens/s (box, max over ranks)", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": value / (BASELINE_TOKENS_PER_S_PER_DEVICE * world),
            "dtype": "bf16", "data": "synthetic uniform token ids, random-init weights",
            "impl": args.impl,
            "config": {"model": ("Llama-3.1-8B" if args.model == "llama3_1_8b" else args.model) if not args.layers else f"{args.model}(layers={args.layers})",
                       "global_batch": args.seqs_per_gpu if cp > 1 else args.seqs_per_gpu * world, "seq_len": S,
                       "parallelism": f"tp{tp}" + ("+sp" if tp > 1 else "") + (f" cp{cp}(zig-zag)" if cp > 1 else "")
                                      + (f" ep{ep}" if ep > 1 else "") + f" dp{dp} distributed-optimizer",
                       "micro_batch": 1, "grad_accum_dtype": "fp32", "recompute_layers": args.recompute,
                       "l2": "working set (weights + activations, >100 GB) far exceeds the 126 MB L2 every step"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "final_loss": loss_val,
            "kernel_status_word": status,
            "gemm_backend": Fn.get_gemm_backend(), "attention_backend": Fn.get_attention_backend(),
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
