"""Mixture-of-experts block: top-k router, dropless token dispatcher, grouped expert FFN, shared experts.

Reference behaviour: ``training_graph/transformer/moe/router.py`` (``TopKRouter`` :78-235: fp32 gating,
softmax/sigmoid scores, optional expert bias and group-limited selection, probability normalisation and
scaling, aux loss), ``token_dispatcher.py`` (:94-347: sort by expert, count exchange, all-to-all-v,
local re-sort, reverse path), ``ffn.py`` (``FFNGroupedGEMM`` :38-168, weights ``weight1 [E,h,2F]`` and
``weight2 [E,F,h]``), ``moe_layer.py`` (:71-156) and ``shared_experts.py`` (:30-124).

Layout used by the kernels: token copies are sorted by (local) expert and every expert segment is
padded to a multiple of 128 rows, so the grouped tcgen05 GEMM maps whole row blocks to experts and
needs no host-side sizes. All index tensors are built on the device.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ...ops import functional as Fn
from .. import mappings as M
from .. import parallel_state as ps
from .mlp import MLP
from .tensor_parallel import default_init
from ...ops.functional import apply_fn

BLOCK = 128  # row block of the grouped GEMM


# ==================================================================================================
# Router
# ==================================================================================================
class TopKRouter(nn.Module):
    """Gating network. ``forward`` returns ``(probs [T,k], expert_ids [T,k], aux_loss | None)``."""

    def __init__(self, config):
        super().__init__()
        self.config = config
        E, H = config.num_moe_experts, config.hidden_size
        dev = getattr(config, "device", None) or ("cuda" if torch.cuda.is_available() else "cpu")
        w = torch.empty(E, H, dtype=torch.float32, device=dev)
        default_init(config.init_method_std)(w)
        self.weight = nn.Parameter(w.to(config.moe_router_dtype))
        self.weight.sequence_parallel = bool(config.sequence_parallel)
        self.weight.no_weight_decay = False
        self.topk = config.moe_router_topk
        self.score_fn = config.moe_router_score_function
        if config.moe_router_enable_expert_bias:
            self.register_buffer("expert_bias", torch.zeros(E, dtype=torch.float32, device=dev))
            self.register_buffer("expert_load", torch.zeros(E, dtype=torch.float32, device=dev), persistent=False)
        else:
            self.expert_bias = None
            self.expert_load = None

    def gating(self, x):
        return F.linear(x.to(self.weight.dtype), self.weight).float()

    def _select(self, scores):
        cfg = self.config
        sel = scores if self.expert_bias is None else scores + self.expert_bias
        T, E = scores.shape
        if cfg.moe_router_num_groups and cfg.moe_router_group_topk and cfg.moe_router_num_groups > 1:
            G = cfg.moe_router_num_groups
            grouped = sel.view(T, G, E // G)
            gscore = grouped.topk(2, dim=-1).values.sum(-1) if self.expert_bias is not None else grouped.max(-1).values
            keep = gscore.topk(cfg.moe_router_group_topk, dim=-1).indices
            mask = torch.zeros(T, G, dtype=torch.bool, device=scores.device).scatter_(1, keep, True)
            sel = sel.masked_fill(~mask.unsqueeze(-1).expand(T, G, E // G).reshape(T, E), float("-inf"))
        ids = sel.topk(self.topk, dim=-1).indices
        return ids

    def forward(self, x: torch.Tensor):
        cfg = self.config
        logits = self.gating(x)
        if cfg.moe_z_loss_coeff:
            z = torch.logsumexp(logits, dim=-1).pow(2).mean() * cfg.moe_z_loss_coeff
        else:
            z = None
        E = cfg.num_moe_experts
        want_aux = self.training and bool(cfg.moe_aux_loss_coeff)
        counts = None
        if self.training and (cfg.moe_aux_loss_coeff or self.expert_load is not None):
            counts = torch.zeros(E, dtype=torch.float32, device=x.device)
        sig = self.score_fn == "sigmoid"
        norm = bool(cfg.norm_topk_prob)
        probs, ids, scores = Fn.router_topk(
            logits, self.expert_bias, self.topk, sigmoid=sig, norm=norm, scale=float(cfg.moe_router_topk_scaling_factor),
            groups=int(cfg.moe_router_num_groups or 0), group_topk=int(cfg.moe_router_group_topk or 0),
            need_scores=want_aux, counts=counts)
        aux = None
        if want_aux:
            T = x.shape[0]
            density = scores.mean(0) if not sig else (scores / (scores.sum(-1, keepdim=True) + 1e-20)).mean(0)
            frac = counts / (T * self.topk)
            aux = cfg.moe_aux_loss_coeff * E * torch.sum(density * frac.detach())
        if z is not None:
            aux = z if aux is None else aux + z
        if self.training and self.expert_load is not None:
            self.expert_load += counts.detach()
        return probs, ids, aux

    @torch.no_grad()
    def update_expert_bias(self, group=None):
        """Aux-loss-free balancing: push the bias of over-loaded experts down (host-free)."""
        if self.expert_bias is None:
            return
        load = self.expert_load.clone()
        if group is not None and dist.is_initialized():
            dist.all_reduce(load, group=group)
        err = load.mean() - load
        self.expert_bias += self.config.moe_router_bias_update_rate * torch.sign(err)
        self.expert_load.zero_()


# ==================================================================================================
# Permutation plan (device-side)
# ==================================================================================================
class PermutePlan:
    """Index tensors that place ``T*k`` token copies into the padded, expert-sorted layout."""

    def __init__(self, expert_ids: torch.Tensor, num_experts: int, rows_bound: Optional[int] = None):
        dev = expert_ids.device
        flat = expert_ids.reshape(-1)
        n = flat.numel()
        self.n = n
        counts = torch.bincount(flat, minlength=num_experts)
        padded = (counts + BLOCK - 1) // BLOCK * BLOCK
        offs = torch.zeros(num_experts + 1, dtype=torch.int64, device=dev)
        offs[1:] = torch.cumsum(padded, 0)
        starts = torch.zeros(num_experts, dtype=torch.int64, device=dev)
        starts[1:] = torch.cumsum(counts, 0)[:-1]
        order = torch.argsort(flat, stable=True)                  # sorted position -> copy index
        sorted_e = flat[order]
        within = torch.arange(n, device=dev) - starts[sorted_e]
        dest_sorted = offs[sorted_e] + within                    # row of each sorted copy
        self.dest = torch.empty(n, dtype=torch.int64, device=dev)
        self.dest[order] = dest_sorted                           # row of copy i (i = t*k + j)
        self.rows = rows_bound if rows_bound is not None else (n + num_experts * (BLOCK - 1) + BLOCK - 1) // BLOCK * BLOCK
        self.counts = counts
        self.group_offsets = offs.to(torch.int32)
        nblocks = self.rows // BLOCK
        blk_start = torch.arange(nblocks, device=dev, dtype=torch.int64) * BLOCK
        self.block_group = (torch.searchsorted(offs[1:].contiguous(), blk_start, right=True)
                            .clamp(max=num_experts - 1).to(torch.int32))
        self.num_blocks = (offs[-1:] // BLOCK).to(torch.int32)


def permute(x: torch.Tensor, plan: PermutePlan, topk: int) -> torch.Tensor:
    """[T,H] → [rows,H]; copy ``t*k+j`` goes to row ``plan.dest[t*k+j]``; padding rows are zero."""
    out = torch.zeros((plan.rows, x.shape[1]), dtype=x.dtype, device=x.device)
    src = torch.arange(plan.n, device=x.device) // topk
    out.index_copy_(0, plan.dest, x.index_select(0, src))
    return out


def unpermute(y: torch.Tensor, plan: PermutePlan, probs: torch.Tensor) -> torch.Tensor:
    """[rows,H] → [T,H] = Σ_j probs[t,j] · y[dest[t,j]]."""
    T, k = probs.shape
    g = y.index_select(0, plan.dest).view(T, k, -1)
    return (g.float() * probs.unsqueeze(-1).float()).sum(1).to(y.dtype)


# ==================================================================================================
# Grouped expert FFN
# ==================================================================================================
class _GroupedLinearFn(torch.autograd.Function):
    """y[rows_g] = x[rows_g] @ W[g] with W ``[G, in, out]`` (the reference's weight1/weight2 layout)."""

    @staticmethod
    def forward(ctx, x, w, block_group, num_blocks, group_offsets):
        from ..recompute import cached_output
        ctx.save_for_backward(x, w, block_group, num_blocks, group_offsets)
        return cached_output(lambda: Fn.grouped_gemm(x, w, block_group, num_blocks, b_mn=True))

    @staticmethod
    def backward(ctx, dy):
        x, w, block_group, num_blocks, group_offsets = ctx.saved_tensors
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = Fn.grouped_gemm(dy, w, block_group, num_blocks, b_mn=False)
        if ctx.needs_input_grad[1]:
            main_grad = getattr(w, "main_grad", None)
            G = w.shape[0]
            if main_grad is not None:
                Fn.grouped_wgrad(x, dy, group_offsets, G, main_grad.view(w.shape), accumulate=True)
            else:
                dw = torch.empty(w.shape, dtype=torch.float32, device=w.device)
                Fn.grouped_wgrad(x, dy, group_offsets, G, dw)
                dw = dw.to(w.dtype)
        return dx, dw, None, None, None


class GroupedMLP(nn.Module):
    """Experts of this rank as two stacked weights: ``weight1 [E_local, H, 2F]``, ``weight2 [E_local, F, H]``."""

    def __init__(self, config, num_local_experts: int):
        super().__init__()
        self.config = config
        self.E = num_local_experts
        H, F_ = config.hidden_size, config.moe_ffn_hidden_size
        dev = getattr(config, "device", None) or ("cuda" if torch.cuda.is_available() else "cpu")
        # draw the weights of all experts from the shared RNG stream, then keep this rank's slice, so the
        # model does not depend on the expert-parallel size
        ep, ep_rank = ps.get_expert_model_parallel_world_size(), ps.get_expert_model_parallel_rank()
        lo, hi = ep_rank * self.E, (ep_rank + 1) * self.E
        # expert tensor parallelism: every expert's FFN width is split over the expert-tensor-parallel ranks (gate and
        # up halves separately); the dispatcher gathers the rows of those ranks before the experts and reduce-scatters
        # the partial outputs after (reference ``modules/transformer/moev3.py:758-850``)
        etp, er = ps.get_expert_tensor_parallel_world_size(), ps.get_expert_tensor_parallel_rank()
        if etp > 1 and F_ % etp:
            raise ValueError(f"moe_ffn_hidden_size {F_} is not divisible by the expert tensor parallel size {etp}")
        self.etp = etp
        Fl = F_ // etp
        w1 = torch.empty(self.E * ep, H, 2 * F_, dtype=torch.float32, device=dev).normal_(0.0, config.init_method_std)
        w1 = w1[lo:hi]
        if etp > 1:
            w1 = torch.cat((w1[..., er * Fl:(er + 1) * Fl], w1[..., F_ + er * Fl:F_ + (er + 1) * Fl]), dim=-1)
        self.weight1 = nn.Parameter(w1.to(config.params_dtype).contiguous())
        del w1
        w2 = torch.empty(self.E * ep, F_, H, dtype=torch.float32, device=dev).normal_(0.0, config.output_layer_init_std)
        w2 = w2[lo:hi]
        if etp > 1:
            w2 = w2[:, er * Fl:(er + 1) * Fl]
        self.weight2 = nn.Parameter(w2.to(config.params_dtype).contiguous())
        del w2
        for p in (self.weight1, self.weight2):
            p.allreduce = False          # reduced over the expert-data-parallel group only
            p.is_expert = True
        if etp > 1:
            self.weight1.tensor_model_parallel, self.weight1.partition_dim = True, 2
            self.weight1.partition_sections = (F_, F_)
            self.weight2.tensor_model_parallel, self.weight2.partition_dim = True, 1
            for p in (self.weight1, self.weight2):
                p.partition_stride = 1

    w1_fp8 = w2_fp8 = w1_scale_inv = w2_scale_inv = None

    def quantize_fp8_(self) -> bool:
        """Inference: replace the bf16 expert weights by block-scaled fp8 ones (``[E, out, in]`` e4m3 with one fp32
        scale per 128 x 128 block, the DeepSeek-V3 checkpoint format)."""
        H, F2 = self.weight1.shape[1], self.weight1.shape[2]
        Fh = self.weight2.shape[1]
        if H % 128 or F2 % 128 or Fh % 128:
            return False
        self.w1_fp8, self.w1_scale_inv = Fn.quantize_weight_128x128(self.weight1.detach().transpose(1, 2).contiguous())
        self.w2_fp8, self.w2_scale_inv = Fn.quantize_weight_128x128(self.weight2.detach().transpose(1, 2).contiguous())
        self._parameters.pop("weight1", None)
        self._parameters.pop("weight2", None)
        self.weight1 = self.weight2 = None
        return True

    def forward(self, x, plan: PermutePlan):
        if self.w1_fp8 is not None:
            # with the segment fill of the plan a call with few rows per expert (decode) takes the kernel that puts
            # the weights on the MMA rows and only the rows in use on the columns
            kw = dict(block_group=plan.block_group, num_blocks=plan.num_blocks,
                      group_offsets=getattr(plan, "group_offsets", None), seg_fill=getattr(plan, "seg_fill", None))
            xq, sa = Fn.quantize_act_1x128(x)
            h = Fn.fp8_gemm(xq, sa, self.w1_fp8, self.w1_scale_inv, **kw)
            hq, sh = Fn.quantize_act_1x128(Fn.swiglu(h))
            return Fn.fp8_gemm(hq, sh, self.w2_fp8, self.w2_scale_inv, **kw)
        h = apply_fn(_GroupedLinearFn, x, self.weight1, plan.block_group, plan.num_blocks, plan.group_offsets)
        h = Fn.swiglu(h)
        return apply_fn(_GroupedLinearFn, h, self.weight2, plan.block_group, plan.num_blocks, plan.group_offsets)


class SharedExpertMLP(MLP):
    """Always-on expert(s); optional sigmoid gate (reference ``shared_experts.py:30-124``)."""

    def __init__(self, config):
        super().__init__(config, ffn_hidden_size=config.moe_shared_expert_intermediate_size)
        if config.use_shared_expert_gating:
            dev = getattr(config, "device", None) or ("cuda" if torch.cuda.is_available() else "cpu")
            self.gate_weight = nn.Parameter(torch.zeros(1, config.hidden_size, dtype=config.params_dtype, device=dev))
            self.gate_weight.sequence_parallel = bool(config.sequence_parallel)
        else:
            self.gate_weight = None

    def forward(self, hidden):
        out, _ = super().forward(hidden)
        if self.gate_weight is not None:
            out = out * torch.sigmoid(F.linear(hidden, self.gate_weight))
        return out


# ==================================================================================================
# Dispatcher + layer
# ==================================================================================================
class MoEAlltoAllTokenDispatcher:
    """Dropless dispatcher over the expert-parallel group (NCCL all-to-all-v baseline path).

    With a single expert-parallel rank no communication and no host synchronisation happens. With
    ``ep > 1`` the split sizes are exchanged first (one small all-to-all and one device→host copy);
    the fused peer-memory kernels in ``parallel/fused_comm.py`` avoid that copy.
    """

    def __init__(self, config):
        self.config = config
        self.ep = ps.get_expert_model_parallel_world_size()
        self.ep_rank = ps.get_expert_model_parallel_rank()
        self.group = ps.get_expert_model_parallel_group()
        self.E = config.num_moe_experts
        self.E_local = self.E // self.ep
        self.k = config.moe_router_topk

    def dispatch(self, x, ids):
        """Returns (expert input in padded layout, plan, context for ``combine``)."""
        T = x.shape[0]
        if self.ep == 1:
            plan = PermutePlan(ids, self.E)
            return permute(x, plan, self.k), plan, ("local", T)
        # 1) order copies by destination rank then expert (global expert id order does both)
        flat = ids.reshape(-1)
        order = torch.argsort(flat, stable=True)
        sorted_e = flat[order]
        send = x.index_select(0, order // self.k)
        counts = torch.bincount(flat, minlength=self.E).view(self.ep, self.E_local)
        recv_counts = torch.empty_like(counts)
        dist.all_to_all_single(recv_counts.view(-1), counts.view(-1).contiguous(), group=self.group)
        in_splits = counts.sum(1).tolist()
        out_splits = recv_counts.sum(1).tolist()
        recv = M.all_to_all(send, out_splits, in_splits, self.group)
        # 2) received copies are (source rank, local expert) ordered; build their local expert ids
        n_recv = recv.shape[0]
        local_e = torch.repeat_interleave(
            torch.arange(self.E_local, device=x.device).repeat(self.ep), recv_counts.view(-1), output_size=n_recv)
        plan = PermutePlan(local_e, self.E_local)
        return permute(recv, plan, 1), plan, ("ep", T, order, in_splits, out_splits)

    def combine(self, y, plan, ctx, probs):
        if ctx[0] == "local":
            return unpermute(y, plan, probs)
        _, T, order, in_splits, out_splits = ctx
        back = y.index_select(0, plan.dest)                    # (source rank, expert) order again
        ret = M.all_to_all(back, in_splits, out_splits, self.group)   # sorted-copy order on the source
        k = self.k
        w = probs.reshape(-1)[order].unsqueeze(-1)
        out = torch.zeros((T, y.shape[1]), dtype=torch.float32, device=y.device)
        out.index_add_(0, order // k, ret.float() * w.float())
        return out.to(y.dtype)


class MoELayer(nn.Module):
    """Router → dispatch → grouped experts → combine (+ shared experts). Returns ``(out, aux_loss)``."""

    def __init__(self, config, layer_number: int = 1, submodules: Optional[dict] = None):
        """``submodules`` (from a layer spec): classes for ``router``, ``experts`` and ``shared_experts``."""
        super().__init__()
        self.config = config
        self.layer_number = layer_number
        sub = submodules or {}
        ep = ps.get_expert_model_parallel_world_size()
        self.router = sub.get("router", TopKRouter)(config)
        self.experts = sub.get("experts", GroupedMLP)(config, config.num_moe_experts // ep)
        self.shared_experts = (sub.get("shared_experts", SharedExpertMLP)(config)
                               if config.moe_shared_expert_intermediate_size else None)
        # the plain all-to-all dispatcher is the default; the all-gather and two-level ("deredundency") dispatchers,
        # safe-token padding and tensor-parallel experts go through the staged dispatcher
        kind = getattr(config, "moe_token_dispatcher_type", "alltoall") or "alltoall"
        if getattr(config, "use_allgather_dispatcher", False):
            kind = "allgather"
        if getattr(config, "enable_deredundency", False):
            kind = "deredundency"
        self.expert_tp = getattr(self.experts, "etp", 1) > 1
        self.staged = kind != "alltoall" or self.expert_tp or bool(getattr(config, "use_pad_tokens", False))
        if self.staged:
            from .moe_dispatchers import StagedTokenDispatcher
            self.dispatcher = StagedTokenDispatcher(config, kind, expert_tp=self.expert_tp)
        else:
            self.dispatcher = MoEAlltoAllTokenDispatcher(config)

    def _tp_sliced(self, hidden):
        """Tensor-parallel attention + expert-parallel MoE without sequence parallelism (the inference layout of the
        reference's DeepSeek-V3 model, ``research/deepseek3/deepseek3_model_infer.py``): every tensor-parallel rank
        holds all tokens, so each one routes only its 1/tp slice of them through the experts and the slices are
        all-gathered afterwards. Tokens are padded to a multiple of tp."""
        tp, rank = ps.get_tensor_model_parallel_world_size(), ps.get_tensor_model_parallel_rank()
        T = hidden.shape[0]
        per = -(-T // tp)
        pad = per * tp - T
        x = torch.nn.functional.pad(hidden, (0, 0, 0, pad)) if pad else hidden
        mine = x[rank * per:(rank + 1) * per].contiguous()
        out, aux = self._forward_local(mine, with_shared=False)
        full = torch.empty((per * tp, out.shape[1]), dtype=out.dtype, device=out.device)
        dist.all_gather_into_tensor(full, out.contiguous(), group=ps.get_tensor_model_parallel_group())
        full = full[:T]
        if self.shared_experts is not None:       # tensor-parallel MLP: runs on all tokens of every rank
            full = full + self.shared_experts(hidden)
        return full, aux

    def forward(self, hidden):
        cfg = self.config
        if (ps.get_tensor_model_parallel_world_size() > 1 and not cfg.sequence_parallel and not self.expert_tp
                and ps.get_expert_model_parallel_world_size() > 1 and not torch.is_grad_enabled()):
            return self._tp_sliced(hidden)
        return self._forward_local(hidden)

    def _forward_local(self, hidden, with_shared: bool = True):
        probs, ids, aux = self.router(hidden)
        from .. import fused_comm
        if not self.staged and fused_comm.moe_enabled(self.config, hidden):
            out = fused_comm.moe_dispatch_experts_combine(self, hidden, probs, ids)
        else:
            x, plan, ctx = self.dispatcher.dispatch(hidden, ids)
            y = self.experts(x, plan)
            out = self.dispatcher.combine(y, plan, ctx, probs.to(hidden.dtype))
        if with_shared and self.shared_experts is not None:
            out = out + self.shared_experts(hidden)
        return out, aux
