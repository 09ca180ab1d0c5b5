"""Worker (torchrun, gloo, CPU): data-parallel attention + expert-parallel MoE inference. Every rank generates for its
own prompts with its own number of new tokens; the experts are split over the ranks, so all ranks step in lockstep
until the slowest is done. Each rank's tokens must equal those of an unsharded model on the same prompts."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mindformers_b200.models import AutoModel  # noqa: E402
from mindformers_b200.parallel import parallel_state as ps  # noqa: E402

CFG = dict(model_type="qwen3_moe", num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
           head_dim=16, intermediate_size=128, moe_intermediate_size=32, num_experts=4, num_experts_per_tok=2,
           vocab_size=128, max_position_embeddings=64, params_dtype="float32", norm_topk_prob=True)


def main():
    out_file = sys.argv[1]
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    g = torch.Generator().manual_seed(3)
    prompts = torch.randint(3, 128, (world, 2, 6), generator=g).tolist()
    new = [3 + 4 * r for r in range(world)]                       # rank 0 finishes long before the last rank
    ps.initialize_model_parallel(tensor_model_parallel_size=1, expert_model_parallel_size=world)
    torch.manual_seed(11)
    model = AutoModel.from_config(dict(CFG, expert_model_parallel_size=world), device="cpu").eval()
    mine = model.generate(prompts[rank], max_new_tokens=new[rank], do_sample=False, eos_token_id=None)
    ps.destroy_model_parallel()
    ps.initialize_model_parallel(tensor_model_parallel_size=1, expert_model_parallel_size=1)
    torch.manual_seed(11)
    full = AutoModel.from_config(CFG, device="cpu").eval()
    ref = full.generate(prompts[rank], max_new_tokens=new[rank], do_sample=False, eos_token_id=None)
    ok = torch.tensor([1 if mine == ref else 0])
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if rank == 0:
        json.dump({"ok": bool(ok.item()), "lens": [len(s) for s in mine]}, open(out_file, "w"))
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok.item() else 1)


if __name__ == "__main__":
    main()
