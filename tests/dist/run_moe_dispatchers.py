"""Worker: every token-dispatcher variant of the MoE layer gives the output and the gradients of a dense loop over the
experts. Launched with 4 gloo ranks: ``--mode ep`` runs expert parallel 4 (all-to-all, all-gather, two-level with 2
ranks per node, each with and without safe tokens); ``--mode etp`` runs tensor parallel 2 x expert parallel 2 with the
experts' FFN width split over the tensor-parallel pair."""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch
import torch.distributed as dist

from mindformers_b200.parallel import parallel_state as ps
from mindformers_b200.parallel.layers.moe import MoELayer
from mindformers_b200.parallel.transformer_config import TransformerConfig

E, K, H, F, T = 8, 2, 32, 48, 24


def make_cfg(**kw):
    cfg = TransformerConfig(num_layers=1, hidden_size=H, num_attention_heads=4, ffn_hidden_size=64, vocab_size=64,
                            seq_length=16, params_dtype="float32", compute_dtype="float32", num_moe_experts=E,
                            moe_router_topk=K, moe_ffn_hidden_size=F, moe_aux_loss_coeff=0.0, init_method_std=0.25, **kw)
    cfg.device = "cpu"
    return cfg


def dense_reference(x, router_w, w1_full, w2_full):
    """Top-k softmax routing and a loop over whole experts, in the layer's conventions (weights renormalised)."""
    logits = x @ router_w.t()
    scores = torch.softmax(logits.float(), dim=-1)
    top, ids = torch.topk(scores, K, dim=-1)
    top = top / top.sum(-1, keepdim=True)
    out = torch.zeros_like(x)
    for e in range(E):
        mask = ids == e
        if not mask.any():
            continue
        rows = mask.any(-1).nonzero().reshape(-1)
        h = x[rows] @ w1_full[e]
        g, u = h.chunk(2, dim=-1)
        y = (torch.nn.functional.silu(g) * u) @ w2_full[e]
        out[rows] += y * (top[rows] * mask[rows]).sum(-1, keepdim=True)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="ep")
    args = ap.parse_args()
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    assert world == 4
    if args.mode == "ep":
        ps.initialize_model_parallel(tensor_model_parallel_size=1, expert_model_parallel_size=4, expert_tensor_parallel_size=1)
        variants = [dict(), dict(use_pad_tokens=True), dict(moe_token_dispatcher_type="allgather"),
                    dict(use_allgather_dispatcher=True, use_pad_tokens=True),
                    dict(enable_deredundency=True, npu_nums_per_device=2),
                    dict(enable_deredundency=True, npu_nums_per_device=2, use_pad_tokens=True)]
        ep, etp = 4, 1
    else:
        ps.initialize_model_parallel(tensor_model_parallel_size=2, expert_model_parallel_size=2)
        variants = [dict(), dict(use_pad_tokens=True), dict(moe_token_dispatcher_type="allgather")]
        ep, etp = 2, 2
    worst = 0.0
    for kw in variants:
        torch.manual_seed(11)                      # the same full-size draws on every rank
        cfg = make_cfg(expert_model_parallel_size=ep, tensor_model_parallel_size=2 if etp > 1 else 1,
                       expert_tensor_parallel_size=etp, **kw)
        layer = MoELayer(cfg)
        assert layer.staged == bool(kw) or etp > 1
        # full weights for the reference: gather the expert shards
        w1, w2 = layer.experts.weight1.detach(), layer.experts.weight2.detach()
        if etp > 1:
            parts1 = [torch.empty_like(w1) for _ in range(etp)]
            parts2 = [torch.empty_like(w2) for _ in range(etp)]
            dist.all_gather(parts1, w1.contiguous(), group=ps.get_expert_tensor_parallel_group())
            dist.all_gather(parts2, w2.contiguous(), group=ps.get_expert_tensor_parallel_group())
            Fl = F // etp
            w1 = torch.cat([p[..., :Fl] for p in parts1] + [p[..., Fl:] for p in parts1], dim=-1)
            w2 = torch.cat(parts2, dim=1)
        g1 = [torch.empty_like(w1) for _ in range(ep)]
        g2 = [torch.empty_like(w2) for _ in range(ep)]
        dist.all_gather(g1, w1.contiguous(), group=ps.get_expert_model_parallel_group())
        dist.all_gather(g2, w2.contiguous(), group=ps.get_expert_model_parallel_group())
        w1_full, w2_full = torch.cat(g1, 0).requires_grad_(), torch.cat(g2, 0).requires_grad_()
        router_w = layer.router.weight.detach().clone().requires_grad_()
        torch.manual_seed(100 + rank)              # every rank routes its own tokens
        x = torch.randn(T, H, requires_grad=True)
        x_ref = x.detach().clone().requires_grad_()
        out, _ = layer(x)
        ref = dense_reference(x_ref, router_w, w1_full, w2_full)
        err = (out - ref).abs().max().item()
        assert ref.abs().max().item() > 1e-4 and out.abs().max().item() > 1e-4, "the comparison is not vacuous"
        gout = torch.randn_like(out)
        out.backward(gout)
        ref.backward(gout)
        gerr = (x.grad - x_ref.grad).abs().max().item()
        # expert-weight gradients: the reference's are for this rank's tokens only; sum them over all ranks and compare
        # this rank's shard
        dist.all_reduce(w1_full.grad)
        dist.all_reduce(w2_full.grad)
        lo = ps.get_expert_model_parallel_rank() * (E // ep)
        ref_g1, ref_g2 = w1_full.grad[lo:lo + E // ep], w2_full.grad[lo:lo + E // ep]
        if etp > 1:
            er, Fl = ps.get_expert_tensor_parallel_rank(), F // etp
            ref_g1 = torch.cat((ref_g1[..., er * Fl:(er + 1) * Fl], ref_g1[..., F + er * Fl:F + (er + 1) * Fl]), dim=-1)
            ref_g2 = ref_g2[:, er * Fl:(er + 1) * Fl]
        my_g1, my_g2 = layer.experts.weight1.grad.clone(), layer.experts.weight2.grad.clone()
        edp_group = ps.get_expert_data_parallel_group()
        if edp_group is not None:
            dist.all_reduce(my_g1, group=edp_group)
            dist.all_reduce(my_g2, group=edp_group)
        werr = max((my_g1 - ref_g1).abs().max().item(), (my_g2 - ref_g2).abs().max().item())
        rerr = (layer.router.weight.grad - router_w.grad).abs().max().item()
        assert router_w.grad.abs().max().item() > 0 and ref_g1.abs().max().item() > 0
        worst = max(worst, err, gerr, werr, rerr)
        if rank == 0:
            print(args.mode, kw, f"|out| {out.abs().max().item():.2e} out {err:.2e} dx {gerr:.2e} dw {werr:.2e} drouter {rerr:.2e}", flush=True)
    t = torch.tensor([worst])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.destroy_process_group()
    sys.exit(0 if t.item() < 5e-5 else 1)


if __name__ == "__main__":
    main()
