"""Pipeline parallelism: how much of the activation send/recv hides behind compute.

Two (or more) pipeline stages, one per GPU, 1F1B schedule over ``--microbatches`` micro-batches of a Llama-shaped
model. The step is timed (CUDA events, max over ranks) with the transfers on their own stream (``overlap``) and on
the compute stream (``serial``); the bytes sent per step and the time they would take alone on the link give the
exposed fraction:  hidden = 1 - (t_overlap - t_ideal) / (t_serial - t_ideal)  with  t_ideal = t_serial - t_comm.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/bench_pipeline_overlap.py
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mindformers_b200.parallel import parallel_state as ps  # noqa: E402
from mindformers_b200.parallel.distributed.optimizer import DistributedOptimizer  # noqa: E402
from mindformers_b200.parallel.layers.gpt_model import GPTModel  # noqa: E402
from mindformers_b200.parallel.pipeline import PipelineTrainStep  # noqa: E402
from mindformers_b200.parallel.transformer_config import TransformerConfig  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--microbatches", type=int, default=8)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    world = int(os.environ["WORLD_SIZE"])
    rank = int(os.environ["RANK"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    ps.initialize_model_parallel(pipeline_model_parallel_size=world)
    cfg = TransformerConfig(num_layers=args.layers, hidden_size=args.hidden, num_attention_heads=args.hidden // 128,
                            num_query_groups=8, ffn_hidden_size=int(args.hidden * 3.5), vocab_size=32000,
                            seq_length=args.seq, max_position_embeddings=args.seq, params_dtype="bfloat16",
                            compute_dtype="bfloat16", pipeline_model_parallel_size=world,
                            untie_embeddings_and_output_weights=True)
    cfg.device = "cuda"
    torch.manual_seed(3)
    pp_rank = ps.get_pipeline_model_parallel_rank()
    model = GPTModel(cfg, pre_process=pp_rank == 0, post_process=pp_rank == world - 1)
    opt = DistributedOptimizer(torch.nn.ModuleList([model]), learning_rate=1e-4, betas=(0.9, 0.95), weight_decay=0.0,
                               max_grad_norm=1.0)
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, 32000, (args.microbatches, args.seq + 1), generator=g).cuda()
    batch = {"input_ids": ids[:, :-1].contiguous(), "labels": ids[:, 1:].contiguous()}

    def timed(overlap):
        step = PipelineTrainStep([model], opt, micro_batch_size=1, overlap=overlap)
        for _ in range(2):
            step(batch)
        dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(args.steps):
            step(batch)
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / args.steps], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    t_overlap = timed(True)
    t_serial = timed(False)
    # activation bytes one stage boundary carries per step: forward + backward, every micro-batch
    bytes_per_step = 2 * args.microbatches * args.seq * args.hidden * 2
    buf = torch.empty(args.seq * args.hidden, dtype=torch.bfloat16, device="cuda")
    for _ in range(2):                      # the first transfer sets up the point-to-point channel
        if rank == 0:
            dist.send(buf, 1)
        elif rank == 1:
            dist.recv(buf, 0)
    dist.barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(2 * args.microbatches):
        if rank == 0:
            dist.send(buf, 1)
        elif rank == 1:
            dist.recv(buf, 0)
    e.record()
    torch.cuda.synchronize()
    t_comm = s.elapsed_time(e)
    res = {"pp": world, "layers": args.layers, "hidden": args.hidden, "seq": args.seq, "microbatches": args.microbatches,
           "ms_per_step_overlap": t_overlap, "ms_per_step_serial": t_serial, "p2p_bytes_per_step": bytes_per_step,
           "p2p_alone_ms": t_comm, "p2p_gb_s": bytes_per_step / t_comm / 1e6,
           "hidden_fraction": (1.0 - max(t_overlap - (t_serial - t_comm), 0.0) / t_comm) if t_comm > 0 else None}
    if rank == 0:
        print(json.dumps(res))
        if args.out:
            with open(args.out, "w") as f:
                json.dump(res, f, indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
