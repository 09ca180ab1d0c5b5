"""Worker (torchrun, one rank per GPU): the fused data-parallel optimizer step (reduce-scatter by peer loads,
AdamW, all-gather by peer stores) against the NCCL reduce-scatter / all-gather path on the same model and data,
then a timing of both on a large flat buffer. Writes a JSON summary from rank 0 to --out."""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mindformers_b200.ops import _lib  # noqa: E402
from mindformers_b200.parallel import parallel_state as ps  # noqa: E402
from mindformers_b200.parallel.distributed.optimizer import DistributedOptimizer  # noqa: E402
from mindformers_b200.trainer.engine import TrainingEngine  # noqa: E402

TINY = dict(model_type="llama", num_hidden_layers=2, hidden_size=256, num_attention_heads=4, num_key_value_heads=2,
            intermediate_size=512, vocab_size=1024, rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=256)


def build(fused):
    torch.manual_seed(11)
    os.environ["MFB_FUSED_DP"] = "1" if fused else "0"
    return TrainingEngine.from_model_config(TINY, seq_length=256, learning_rate=1e-3, weight_decay=0.1, max_grad_norm=1.0)


def time_step(opt, iters=5):
    for _ in range(2):
        opt.step(grad_scale=1.0)
    dist.barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        opt.step(grad_scale=1.0)
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    ap.add_argument("--big", type=int, default=256, help="millions of parameters of the timing buffer (0 = skip)")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    ps.initialize_model_parallel(tensor_model_parallel_size=1)
    res = {"dp": world}
    fused, plain = build(True), build(False)
    assert fused.optimizer.fused_dp and not plain.optimizer.fused_dp
    assert all(getattr(sh, "fused", False) for sh in fused.optimizer.shards.values())
    g = torch.Generator().manual_seed(100 + rank)
    worst, losses = 0.0, []
    for step in range(4):
        ids = torch.randint(0, 1024, (2, 257), generator=g).cuda()
        batch = {"input_ids": ids[:, :-1].contiguous(), "labels": ids[:, 1:].contiguous()}
        a = fused.train_step_device(batch)
        b = plain.train_step_device(batch)
        losses.append((float(a["loss"]), float(b["loss"])))
        for (n, p), (_, q) in zip(fused.model.named_parameters(), plain.model.named_parameters()):
            worst = max(worst, (p.float() - q.float()).abs().max().item())
        gn = abs(float(a["global_norm"]) - float(b["global_norm"]))
        worst = max(worst, gn / max(float(b["global_norm"]), 1e-6) * 1e-3)
    # replicas must hold identical parameters after the peer-store all-gather
    flat = torch.cat([p.detach().float().reshape(-1) for p in fused.model.parameters()])
    ref = flat.clone()
    dist.broadcast(ref, src=0)
    res["replica_mismatch"] = float((flat - ref).abs().max())
    res["max_param_diff_vs_nccl"] = worst
    res["losses"] = losses
    res["status"] = _lib.read_status()
    if args.big:
        n = args.big * 1000 * 1000 // (4096 * world) * (4096 * world)
        timings = {}
        for name, flag in (("fused", True), ("nccl", False)):
            lin = torch.nn.Linear(4096, n // 4096, bias=False, device="cuda", dtype=torch.bfloat16)
            opt = DistributedOptimizer(lin, learning_rate=1e-4, weight_decay=0.1, fused_dp_comm=flag)
            for buf in opt.buffers.values():
                buf.grad_data.normal_(0, 1e-3)
            timings[name + "_ms"] = time_step(opt)
            del opt, lin
            torch.cuda.empty_cache()
        shard_bytes = n // world
        # per rank: (world-1)/world of the fp32 gradient slice sums cross NVLink inbound, and (world-1) copies of
        # the bf16 slice outbound; HBM: grad slice read + m, v, lo, p read/write
        nvlink_in = (world - 1) * shard_bytes * 4
        nvlink_out = (world - 1) * shard_bytes * 2
        timings.update(params=n, nvlink_in_bytes=nvlink_in, nvlink_out_bytes=nvlink_out,
                       nvlink_floor_ms=max(nvlink_in, nvlink_out) / 770e9 * 1e3,
                       hbm_bytes=shard_bytes * (4 * world + 4 + 8 + 8 + 4 + 4 + 2 * world),
                       hbm_floor_ms=shard_bytes * (4 * world + 4 + 8 + 8 + 4 + 4 + 2 * world) / 6523.7e9 * 1e3)
        res["bench"] = timings
        res["status_after_bench"] = _lib.read_status()
    if rank == 0:
        print(json.dumps(res, indent=1))
        if args.out:
            with open(args.out, "w") as f:
                json.dump(res, f, indent=1)
    ok = res["status"] == 0 and res["replica_mismatch"] == 0.0 and res["max_param_diff_vs_nccl"] < 1e-2
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
