"""Worker script: trains a tiny model for a few steps under a given parallel layout (gloo, CPU fp32)
and, on rank 0, writes the losses and a digest of the final parameters to --out (JSON).

Launched by tests/test_parallel_cpu.py through torch.distributed.run.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mindformers_b200.parallel import parallel_state as ps  # noqa: E402
from mindformers_b200.parallel.distributed.optimizer import DistributedOptimizer  # noqa: E402
from mindformers_b200.parallel.distributed.train_step import TrainOneStep  # noqa: E402
from mindformers_b200.parallel.layers.gpt_model import GPTModel  # noqa: E402
from mindformers_b200.parallel.transformer_config import TransformerConfig  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--cp", type=int, default=1)
    ap.add_argument("--ep", type=int, default=1)
    ap.add_argument("--sp", type=int, default=0)
    ap.add_argument("--moe", type=int, default=0)
    ap.add_argument("--cp-type", default="all_gather")
    ap.add_argument("--zigzag", type=int, default=0, help="rank r holds sequence chunks r and 2*cp-1-r")
    ap.add_argument("--ulysses", type=int, default=1, help="ulysses_degree_in_cp of the a2a+p2p layout")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--kv-groups", type=int, default=2)
    ap.add_argument("--forward-only", type=int, default=0, help="no training: write the loss of one forward pass")
    ap.add_argument("--out", required=True)
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        dist.init_process_group("gloo")
    ps.initialize_model_parallel(tensor_model_parallel_size=args.tp, context_parallel_size=args.cp,
                                 expert_model_parallel_size=args.ep, expert_tensor_parallel_size=1 if args.moe else None)
    torch.manual_seed(7)
    kw = dict(num_layers=2, hidden_size=64, num_attention_heads=4, num_query_groups=args.kv_groups, ffn_hidden_size=128,
              vocab_size=256, seq_length=32, max_position_embeddings=32, params_dtype="float32",
              compute_dtype="float32", use_scaled_init=False, pad_token_id=-1,
              tensor_model_parallel_size=args.tp, sequence_parallel=bool(args.sp), context_parallel_size=args.cp,
              expert_model_parallel_size=args.ep, cp_comm_type=args.cp_type if args.cp > 1 else None,
              cp_zigzag=bool(args.zigzag), ulysses_degree_in_cp=args.ulysses)
    if args.moe:
        kw.update(num_moe_experts=4, moe_router_topk=2, moe_ffn_hidden_size=32, moe_aux_loss_coeff=1e-2,
                  expert_tensor_parallel_size=1)
    cfg = TransformerConfig(**kw)
    cfg.device = "cpu"
    model = GPTModel(cfg)
    if args.forward_only:
        g = torch.Generator().manual_seed(99)
        ids = torch.randint(0, 256, (4, 33), generator=g)
        with torch.no_grad():
            loss = model.eval()(ids[:, :-1].contiguous(), labels=ids[:, 1:].contiguous())
        if int(os.environ.get("RANK", "0")) == 0:
            with open(args.out, "w") as f:
                json.dump({"losses": [float(loss)], "digest": {}, "norm": 0.0}, f)
        if world > 1:
            dist.barrier()          # no rank tears the group down while another is still inside a collective
            dist.destroy_process_group()
        return
    opt = DistributedOptimizer(model, learning_rate=1e-2, betas=(0.9, 0.95), weight_decay=0.01, max_grad_norm=1.0,
                               sequence_parallel=bool(args.sp))
    step = TrainOneStep(model, opt, micro_batch_size=1)
    g = torch.Generator().manual_seed(99)
    global_batch = 4
    ids_all = torch.randint(0, 256, (global_batch, 33), generator=g)
    dp = ps.get_data_parallel_world_size()
    dpr = ps.get_data_parallel_rank()
    per = global_batch // dp
    ids = ids_all[dpr * per:(dpr + 1) * per]
    inp, lab = ids[:, :-1].contiguous(), ids[:, 1:].contiguous()
    pos = None
    if args.cp > 1:
        cpr = ps.get_context_parallel_rank()
        S = inp.shape[1] // args.cp
        if args.zigzag:
            half = S // 2
            idx = torch.cat((torch.arange(cpr * half, (cpr + 1) * half),
                             torch.arange((2 * args.cp - 1 - cpr) * half, (2 * args.cp - cpr) * half)))
        else:
            idx = torch.arange(cpr * S, (cpr + 1) * S)
        pos = idx.unsqueeze(0).expand(per, S).contiguous()
        inp, lab = inp[:, idx].contiguous(), lab[:, idx].contiguous()
    losses = []
    for _ in range(args.steps):
        batch = {"input_ids": inp, "labels": lab}
        if pos is not None:
            batch["position_ids"] = pos
        out = step(batch)
        loss = out["loss"].clone()
        if world > 1:
            dist.all_reduce(loss, group=ps.get_data_parallel_group(with_context_parallel=True))
            loss /= ps.get_data_parallel_world_size(with_context_parallel=True)
        losses.append(loss.item())
    # digest over parameters that are identical on every rank and every layout
    digest = {}
    for n, p in model.named_parameters():
        if "layernorm" in n or "router" in n:
            digest[n] = p.detach().double().sum().item()
    if int(os.environ.get("RANK", "0")) == 0:
        with open(args.out, "w") as f:
            json.dump({"losses": losses, "digest": digest, "norm": out["global_norm"].item()}, f)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
