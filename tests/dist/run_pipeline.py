"""Worker (gloo on CPU, or NCCL on GPUs): trains a tiny 4-layer model under pipeline parallelism (optionally with
virtual stages) for a few steps and writes losses and a parameter digest from the last stage to --out (JSON)."""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mindformers_b200.parallel import parallel_state as ps  # noqa: E402
from mindformers_b200.parallel.distributed.optimizer import DistributedOptimizer  # noqa: E402
from mindformers_b200.parallel.layers.gpt_model import GPTModel  # noqa: E402
from mindformers_b200.parallel.pipeline import PipelineTrainStep  # noqa: E402
from mindformers_b200.parallel.transformer_config import TransformerConfig  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--vpp", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--moe", type=int, default=0)
    ap.add_argument("--out", required=True)
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    cuda = torch.cuda.is_available() and torch.cuda.device_count() >= world
    if cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    if world > 1:
        dist.init_process_group("nccl" if cuda else "gloo")
    ps.initialize_model_parallel(pipeline_model_parallel_size=args.pp,
                                 virtual_pipeline_model_parallel_size=args.vpp if args.vpp > 1 else None)
    kw = dict(num_layers=4, hidden_size=64, num_attention_heads=4, num_query_groups=2, ffn_hidden_size=128, vocab_size=256,
              seq_length=32, max_position_embeddings=32, params_dtype="float32", compute_dtype="float32", use_scaled_init=False,
              pad_token_id=-1, pipeline_model_parallel_size=args.pp, untie_embeddings_and_output_weights=True,
              virtual_pipeline_model_parallel_size=args.vpp if args.vpp > 1 else None)
    if args.moe:
        kw.update(num_moe_experts=4, moe_router_topk=2, moe_ffn_hidden_size=32, moe_aux_loss_coeff=1e-2)
    cfg = TransformerConfig(**kw)
    cfg.device = "cuda" if cuda else "cpu"
    pp_rank = ps.get_pipeline_model_parallel_rank()
    chunks = []
    # every rank draws the parameters of all layers from the same stream so that the layout does not change them
    for c in range(args.vpp):
        torch.manual_seed(7)
        ps.set_virtual_pipeline_model_parallel_rank(c if args.vpp > 1 else None)
        pre = pp_rank == 0 and c == 0
        post = pp_rank == args.pp - 1 and c == args.vpp - 1
        chunks.append(GPTModel(cfg, pre_process=pre, post_process=post, vp_stage=c if args.vpp > 1 else None))
    # overwrite with the weights of a reference full model built from one seed
    ps_state = ps.get_state()
    sizes = dict(ps_state.sizes)
    ps_state.sizes["pp"] = 1
    ref_cfg = TransformerConfig(**{**kw, "pipeline_model_parallel_size": 1, "virtual_pipeline_model_parallel_size": None})
    ref_cfg.device = cfg.device
    torch.manual_seed(7)
    saved_groups = ps_state.groups["pp"]
    ps_state.groups["pp"] = type(saved_groups)([ps_state.rank])
    ref = GPTModel(ref_cfg)
    ps_state.groups["pp"] = saved_groups
    ps_state.sizes.update(sizes)
    ref_sd = dict(ref.named_parameters())
    with torch.no_grad():
        for ch in chunks:
            for n, p in ch.named_parameters():
                p.copy_(ref_sd[n])          # layers carry their global number on every stage
    del ref
    net = torch.nn.ModuleList(chunks)
    opt = DistributedOptimizer(net, learning_rate=1e-2, betas=(0.9, 0.95), weight_decay=0.01, max_grad_norm=1.0)
    step = PipelineTrainStep(chunks, opt, micro_batch_size=1, overlap=True)
    g = torch.Generator().manual_seed(99)
    ids = torch.randint(0, 256, (4, 33), generator=g).to(cfg.device)
    batch = {"input_ids": ids[:, :-1].contiguous(), "labels": ids[:, 1:].contiguous()}
    losses = []
    for _ in range(args.steps):
        out = step(batch)
        losses.append(float(out["loss"]))
    digest = {}
    for ch in chunks:
        for n, p in ch.named_parameters():
            if "layernorm" in n and ".layers." in n:
                digest[n] = p.detach().double().sum().item()
    gathered = [None] * world
    if world > 1:
        dist.all_gather_object(gathered, digest)
    else:
        gathered = [digest]
    merged = {}
    for d in gathered:
        merged.update(d)
    if int(os.environ.get("RANK", "0")) == 0:
        with open(args.out, "w") as f:
            json.dump({"losses": losses, "digest": merged, "norm": float(out["global_norm"])}, f)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
