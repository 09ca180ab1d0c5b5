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


def build(fused, overlap=True, cfg=None, seq=256, publish=False, **kw):
    torch.manual_seed(11)
    os.environ["MFB_FUSED_DP"] = "1" if fused else "0"
    os.environ["MFB_DP_OVERLAP"] = "1" if overlap else "0"
    os.environ["MFB_DP_PARAM_OVERLAP"] = "1" if publish else "0"
    kw.setdefault("max_grad_norm", 1.0)
    return TrainingEngine.from_model_config(cfg or TINY, seq_length=seq, learning_rate=1e-3, weight_decay=0.1, **kw)


def overlap_timeline(rank, world):
    """Step time with the bucketed reduction under the backward pass and with one reduction after it, and (rank 0,
    torch.profiler) how much of the bucket kernels' time lies before the last backward kernel of the step."""
    cfg = dict(TINY, num_hidden_layers=8, hidden_size=2048, num_attention_heads=16, num_key_value_heads=4,
               intermediate_size=8192, vocab_size=32768, max_position_embeddings=2048)
    out = {}
    g = torch.Generator().manual_seed(5 + rank)
    ids = torch.randint(0, 32768, (4, 2049), generator=g).cuda()
    batch = {"input_ids": ids[:, :-1].contiguous(), "labels": ids[:, 1:].contiguous()}
    for tag, ov in (("overlap", True), ("after_backward", False)):
        eng = build(True, overlap=ov, cfg=cfg, seq=2048, micro_batch_size=2)
        assert bool(eng.optimizer._ov_layers) and eng.optimizer.overlap_grad_reduce == ov
        for _ in range(3):
            eng.train_step_device(batch)
        dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(5):
            eng.train_step_device(batch)
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / 5], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out[tag + "_step_ms"] = round(t.item(), 3)
        if ov:
            from torch.profiler import ProfilerActivity, profile
            with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
                eng.train_step_device(batch)
                torch.cuda.synchronize()
            ks = [ev for ev in prof.events() if ev.device_type == torch.autograd.DeviceType.CUDA]
            red = [ev for ev in ks if "dp_reduce_kernel<false>" in ev.name or "dp_reduce_kernel<(bool)0>" in ev.name]
            bwd = [ev for ev in ks if "gemm" in ev.name or "flash_attn_bwd" in ev.name]
            closing = [ev for ev in ks if "dp_reduce_kernel<true>" in ev.name or "dp_reduce_kernel<(bool)1>" in ev.name]
            if red and bwd and closing:
                last_bwd_end = max(ev.time_range.end for ev in bwd if ev.time_range.end <= closing[0].time_range.start)
                under = sum(min(ev.time_range.end, last_bwd_end) - min(ev.time_range.start, last_bwd_end) for ev in red)
                out["bucket_kernels"] = len(red)
                out["bucket_kernel_us"] = round(sum(ev.time_range.end - ev.time_range.start for ev in red), 1)
                out["bucket_kernel_us_under_backward"] = round(under, 1)
                out["closing_reduce_us"] = round(sum(ev.time_range.end - ev.time_range.start for ev in closing), 1)
        del eng
        torch.cuda.empty_cache()
    return out


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
    ap.add_argument("--timeline", action="store_true", help="time a mid-size model with and without the overlap")
    ap.add_argument("--big", type=int, default=256, help="millions of parameters of the timing buffer (0 = skip)")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    ps.initialize_model_parallel(tensor_model_parallel_size=1)
    res = {"dp": world}
    four = dict(TINY, num_hidden_layers=4)
    fused, plain, serial = build(True, cfg=four), build(False, cfg=four), build(True, overlap=False, cfg=four)
    deferred = build(True, cfg=four, publish=True)      # AdamW + publication under the next forward pass
    assert deferred.optimizer.overlap_param_gather and not fused.optimizer.overlap_param_gather
    deferred_diff = 0.0
    assert fused.optimizer.fused_dp and not plain.optimizer.fused_dp and serial.optimizer.fused_dp
    assert fused.optimizer._ov_layers and fused.optimizer.overlap_grad_reduce and not serial.optimizer.overlap_grad_reduce
    grad_mismatch, serial_param_diff = 0.0, 0.0
    assert all(getattr(sh, "fused", False) for sh in fused.optimizer.shards.values())
    g = torch.Generator().manual_seed(100 + rank)
    worst, losses = 0.0, []
    for step in range(4):
        ids = torch.randint(0, 1024, (2, 257), generator=g).cuda()
        batch = {"input_ids": ids[:, :-1].contiguous(), "labels": ids[:, 1:].contiguous()}
        if step:      # same weights in: the reduced gradients of the bucketed and the single pass must agree bit for bit
            for p, q in zip(serial.model.parameters(), fused.model.parameters()):
                p.data.copy_(q.data)
            for (_, s1), (_, s2) in zip(serial.optimizer.shards.items(), fused.optimizer.shards.items()):
                s1.m.copy_(s2.m), s1.v.copy_(s2.v), s1.lo.copy_(s2.lo)
            serial.optimizer.global_step = fused.optimizer.global_step
        a = fused.train_step_device(batch)
        b = plain.train_step_device(batch)
        c = serial.train_step_device(batch)
        d = deferred.train_step_device(batch)
        assert deferred.optimizer._pub is not None          # the publication is still pending after the step
        if step == 1:
            with torch.no_grad():                           # a forward pass outside the training step waits by itself
                deferred.model(batch["input_ids"][:1], batch["labels"][:1])
        elif step == 2:
            deferred.optimizer.finish_param_gather()
        # step 0: nothing waits here, the next training step's zero_grad / forward pass pick the waits up;
        # step 3: model_state (what a checkpoint calls) waits
        deferred_diff = max(deferred_diff, abs(float(d["loss"]) - float(a["loss"])))
        if step:
            from mindformers_b200.checkpoint.io import model_state
            got = model_state(deferred.model)
            for (n, p) in fused.model.named_parameters():
                deferred_diff = max(deferred_diff, (p.float() - got[n].float()).abs().max().item())
        for (_, s1), (_, s2) in zip(serial.optimizer.shards.items(), fused.optimizer.shards.items()):
            grad_mismatch = max(grad_mismatch, (s1.grad - s2.grad).abs().max().item())
        for p, q in zip(serial.model.parameters(), fused.model.parameters()):
            serial_param_diff = max(serial_param_diff, (p.float() - q.float()).abs().max().item())
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
    res["bucketed_vs_single_pass_grad_mismatch"] = grad_mismatch
    res["bucketed_vs_single_pass_param_diff"] = serial_param_diff
    res["deferred_publication_param_and_loss_diff"] = deferred_diff
    if args.timeline:
        res["timeline"] = overlap_timeline(rank, world)
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
    ok = res["status"] == 0 and res["replica_mismatch"] == 0.0 and res["max_param_diff_vs_nccl"] < 1e-2 \
        and res["bucketed_vs_single_pass_grad_mismatch"] == 0.0 and res["bucketed_vs_single_pass_param_diff"] < 1e-3 \
        and res["deferred_publication_param_and_loss_diff"] == 0.0
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
