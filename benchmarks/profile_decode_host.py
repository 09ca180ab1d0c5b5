"""Host-side profile of the decode loop: ``cProfile`` around 40 greedy decode steps of a DeepSeek-V3-shaped model
(4 layers, 32 experts, fp8 weights, 64 sequences). Shows where Python time goes between kernel launches; the profiler
roughly doubles Python time, so read shares, not absolutes.

    python benchmarks/profile_decode_host.py                                  # one GPU
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/profile_decode_host.py
                                                                              # tp 2 attention + ep 2 experts

Writes ``decode_host_profile_{tottime,cumulative}.txt`` into ``--out`` (rank 0).
"""
import argparse
import cProfile
import io
import os
import pstats
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=".")
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--prompt", type=int, default=256)
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    from mindformers_b200.inference.fp8 import quantize_model_fp8
    from mindformers_b200.models import AutoModel
    from mindformers_b200.models.presets import get_preset
    from mindformers_b200.ops import _lib
    from mindformers_b200.parallel import parallel_state as ps
    cfg = get_preset("deepseek_v3")
    cfg["num_hidden_layers"] = 4
    cfg["n_routed_experts"] = 32
    cfg.pop("num_nextn_predict_layers", None)
    extra = dict(block_size=128, seq_length=args.prompt + args.steps + 8, max_position_embeddings=4096)
    if world > 1:
        ps.initialize_model_parallel(tensor_model_parallel_size=world, expert_model_parallel_size=world,
                                     expert_tensor_parallel_size=1)
        extra.update(tensor_model_parallel_size=world, expert_model_parallel_size=world, expert_tensor_parallel_size=1,
                     fused_tp_comm=True)
    else:
        ps.initialize_model_parallel()
    torch.manual_seed(1)
    model = AutoModel.from_config(cfg, device="cuda", **extra).eval()
    quantize_model_fp8(model)
    g = torch.Generator().manual_seed(7)
    prompts = torch.randint(3, cfg["vocab_size"], (64, args.prompt), generator=g).tolist()
    kw = dict(do_sample=False, eos_token_id=None)
    model.generate(prompts, max_new_tokens=4, **kw)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    prof = cProfile.Profile()
    prof.enable()
    model.generate(prompts, max_new_tokens=args.steps, **kw)
    torch.cuda.synchronize()
    prof.disable()
    if rank == 0:
        os.makedirs(args.out, exist_ok=True)
        for key in ("tottime", "cumulative"):
            s = io.StringIO()
            pstats.Stats(prof, stream=s).sort_stats(key).print_stats(60)
            with open(os.path.join(args.out, f"decode_host_profile_{key}.txt"), "w") as f:
                f.write(s.getvalue())
        print("kernel status word", _lib.read_status())
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
