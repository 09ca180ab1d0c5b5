"""Per-kernel device-time shares of one training step (torch.profiler, rank 0), for this repository's path and for the
library path (cuBLAS + SDPA + NCCL) on the same engine.

    python benchmarks/step_kernel_shares.py --layers 8
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/step_kernel_shares.py --layers 8

The model is Llama-3.1-8B with ``--layers`` layers (shares, not absolute times, are what this is for: the profiler
serialises little but adds launch overhead). Tensor parallel 2 with sequence parallelism from two ranks on.
"""
import argparse
import json
import os
import sys
from collections import defaultdict

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--seqs", type=int, default=4)
    ap.add_argument("--micro-batch", type=int, default=None)
    ap.add_argument("--out", default=None)
    ap.add_argument("--bands", type=int, default=0, help="also time the step with fixed raster bands (A/B)")
    ap.add_argument("--profiled-steps", type=int, default=1, help="consecutive steps inside one profiler session")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from mindformers_b200.models.presets import get_preset
    from mindformers_b200.ops import functional as Fn
    from mindformers_b200.parallel import fused_comm, parallel_state as ps
    from mindformers_b200.trainer.engine import TrainingEngine
    tp = 2 if world >= 2 else 1
    ps.initialize_model_parallel(tensor_model_parallel_size=tp)
    dp = world // tp
    preset = get_preset("llama3_1_8b")
    preset["num_hidden_layers"] = args.layers
    mbs = args.micro_batch or (2 if world >= 2 else 1)
    engine = TrainingEngine.from_model_config(preset, parallel=dict(tensor_model_parallel_size=tp, sequence_parallel=tp > 1),
                                              seq_length=4096, micro_batch_size=mbs)
    n = args.seqs * world // dp
    ids = torch.randint(0, preset["vocab_size"], (n, 4097), device="cuda")
    batch = {"input_ids": ids[:, :-1].contiguous(), "labels": ids[:, 1:].contiguous()}

    def shares(label):
        for _ in range(2):
            engine.train_step_device(batch)
        torch.cuda.synchronize()
        # wall time of a step on the device without the profiler: kernel time / this = how busy the GPU is
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            engine.train_step_device(batch)
        e1.record()
        torch.cuda.synchronize()
        step_ms = e0.elapsed_time(e1) / 3
        with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CUDA]) as prof:
            for _ in range(args.profiled_steps):
                engine.train_step_device(batch)
            torch.cuda.synchronize()
        agg = defaultdict(lambda: [0, 0.0])
        for ev in prof.events():
            if ev.device_type == torch.autograd.DeviceType.CUDA:
                name = ev.name.split("(")[0][:90]
                agg[name][0] += 1
                agg[name][1] += ev.device_time if hasattr(ev, "device_time") else ev.cuda_time
        total = sum(v[1] for v in agg.values())
        # idle time between consecutive kernels, by the kernel that follows the gap: where the host falls behind
        devs = sorted((ev for ev in prof.events() if ev.device_type == torch.autograd.DeviceType.CUDA),
                      key=lambda ev: ev.time_range.start)
        gaps = defaultdict(lambda: [0, 0.0])
        end_prev, name_prev = None, None
        for ev in devs:
            if end_prev is not None:
                gap = ev.time_range.start - end_prev
                if gap > 3.0:
                    key = f"{name_prev.split('(')[0][:50]} -> {ev.name.split('(')[0][:50]}"
                    gaps[key][0] += 1
                    gaps[key][1] += gap
            if end_prev is None or ev.time_range.end > end_prev:
                end_prev, name_prev = ev.time_range.end, ev.name
        gap_rows = sorted(((k, c, t) for k, (c, t) in gaps.items()), key=lambda r: -r[2])
        span_ms = (max(ev.time_range.end for ev in devs) - devs[0].time_range.start) / 1e3
        rows = sorted(((k, c, t) for k, (c, t) in agg.items()), key=lambda r: -r[2])
        if rank == 0:
            print(f"== {label}: {total / 1e3:.1f} ms of kernel time in one step of {step_ms:.1f} ms "
                  f"({args.layers} layers, tp{tp}, mbs {mbs})")
            for k, c, t in rows[:28]:
                print(f"{100 * t / total:6.2f} %  {t / 1e3:9.2f} ms  x{c:<5d} {k}")
        if rank == 0:
            print(f"-- {args.profiled_steps} profiled step(s): first kernel start to last kernel end {span_ms:.1f} ms, "
                  f"kernel time {total / 1e3:.1f} ms")
            print(f"-- idle gaps > 3 us: {sum(t for _, _, t in gap_rows) / 1e3:.1f} ms in {sum(c for _, c, _ in gap_rows)} gaps")
            for k, c, t in gap_rows[:14]:
                print(f"   {t / 1e3:7.2f} ms  x{c:<4d} {k}")
        return {"label": label, "total_ms": total / 1e3, "step_ms": step_ms, "profiled_steps": args.profiled_steps, "span_ms": span_ms,
                "gaps": [(k, c, t / 1e3) for k, c, t in gap_rows[:40]], "rows": [(k, c, t / 1e3) for k, c, t in rows[:60]]}

    out = []
    if args.bands:
        # A/B of the raster band (plain CTA-pair GEMM, tensor-parallel GEMMs) inside the same process and clocks
        import ctypes
        from mindformers_b200.ops import _lib
        lib = _lib.get_lib()
        lib.mfb_tp_set_band.argtypes = [ctypes.c_int]
        lib.mfb_tp_set_band.restype = None
        for plain, tpb in ((8, 8), (16, 8), (0, 8), (0, 16), (0, 0), (8, 8)):
            lib.mfb_gemm_pair_set_band(plain)
            lib.mfb_tp_set_band(tpb)
            out.append(shares(f"this repository, band plain={plain} tp={tpb} (0 = chosen from K)"))
        lib.mfb_gemm_pair_set_band(0)
        lib.mfb_tp_set_band(0)
    out.append(shares("this repository"))
    Fn.set_gemm_backend("cublas")
    Fn.set_attention_backend("sdpa")
    fused_comm.set_enabled(False)
    engine.optimizer.set_fused_dp(False)
    out.append(shares("library path"))
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            json.dump(out, f, indent=1)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
