"""Worker (torchrun, one rank per GPU): a small DeepSeek-V3-shaped model with tensor-parallel attention and
expert-parallel MoE (both over all ranks), bf16 and block-scaled fp8 weights. Checks that generation runs through the
tp-sliced MoE path, that every rank produces the same tokens, that fp8 and bf16 agree on most greedy tokens and that
no bounded device wait ran out. The decode step is also replayed from a CUDA graph (NCCL collectives and the expert
exchange kernels inside the graph) and must give the tokens of the eager run."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mindformers_b200.inference.fp8 import quantize_model_fp8  # noqa: E402
from mindformers_b200.models import AutoModel  # noqa: E402
from mindformers_b200.ops import _lib  # noqa: E402
from mindformers_b200.parallel import parallel_state as ps  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    ps.initialize_model_parallel(tensor_model_parallel_size=world, expert_model_parallel_size=world,
                                 expert_tensor_parallel_size=1)
    cfg = dict(model_type="deepseek_v3", num_hidden_layers=3, hidden_size=1024, num_attention_heads=8,
               num_key_value_heads=8, intermediate_size=2048, moe_intermediate_size=256, n_routed_experts=16,
               n_shared_experts=1, num_experts_per_tok=4, n_group=4, topk_group=2, routed_scaling_factor=1.0,
               norm_topk_prob=True, scoring_func="sigmoid", first_k_dense_replace=1, vocab_size=2048,
               q_lora_rank=512, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
               max_position_embeddings=1024, moe_router_enable_expert_bias=True, block_size=128,
               tensor_model_parallel_size=world, expert_model_parallel_size=world, expert_tensor_parallel_size=1,
               fused_tp_comm=True)
    torch.manual_seed(11)
    model = AutoModel.from_config(cfg, device="cuda").eval()
    g = torch.Generator().manual_seed(5)
    prompts = torch.randint(3, 2048, (4, 256), generator=g).tolist()
    kw = dict(max_new_tokens=8, do_sample=False, eos_token_id=None)
    out_bf16 = model.generate(prompts, **kw)
    stats = quantize_model_fp8(model)
    out_fp8 = model.generate(prompts, **kw)
    out_graph = model.generate(prompts, use_cuda_graph=True, **kw)
    out_graph2 = model.generate(prompts, use_cuda_graph=True, **kw)       # a second capture and replay sequence
    graph_same = out_graph == out_fp8 and out_graph2 == out_fp8
    new_bf16 = torch.tensor([o[256:] for o in out_bf16], device="cuda")
    new_fp8 = torch.tensor([o[256:] for o in out_fp8], device="cuda")
    both = torch.stack([new_bf16, new_fp8])
    gathered = [torch.empty_like(both) for _ in range(world)]
    dist.all_gather(gathered, both)
    same_across_ranks = all(torch.equal(t, gathered[0]) for t in gathered)
    agree = (new_bf16[:, 0] == new_fp8[:, 0]).float().mean().item()       # first generated token of every prompt
    status = _lib.read_status()
    res = {"same_across_ranks": same_across_ranks, "first_token_agreement_fp8_vs_bf16": agree, "status": status,
           "fp8_layers": stats["linear"], "fp8_grouped": stats["grouped"], "graph_matches_eager": graph_same}
    if rank == 0:
        print(json.dumps(res))
    ok = graph_same and same_across_ranks and status == 0 and stats["linear"] > 0 and stats["grouped"] > 0 and agree >= 0.5
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
