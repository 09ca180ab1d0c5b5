"""Capacity-based mixture of experts of the legacy stack (``mindformers/modules/transformer/moe.py``): ``MoEConfig`` :88,
``TopkRouterV2`` :1210 with k-drop / s-drop token dropping (:1623-1770) and expert / device / comm aux losses
(:1794-1887), ``MoEV2`` :635. Tokens above ``capacity = ceil(capacity_factor * tokens * k / experts)`` are dropped (their
expert output is zero, the residual path carries them); everything is batched, no host synchronisation."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class MoEConfig:
    """Legacy MoE settings (reference ``modules/transformer/moe.py:88``): expert count, capacity factor, experts per
    token, drop policy, auxiliary-loss kinds and factors, shared experts, group-limited routing."""

    expert_num: int = 1
    capacity_factor: float = 1.1
    aux_loss_factor: float = 0.05
    num_experts_chosen: int = 1
    expert_group_size: Optional[int] = None
    enable_sdrop: bool = False
    routing_policy: str = "TopkRouterV2"
    norm_topk_prob: bool = True
    router_dense_type: str = "float32"
    shared_expert_num: int = 0
    use_shared_expert_gating: bool = False
    moe_intermediate_size: int = 1407
    routed_scaling_factor: float = 1.0
    aux_loss_types: List[str] = field(default_factory=lambda: ["expert"])
    aux_loss_factors: List[float] = field(default_factory=lambda: [0.05])
    z_loss_factor: float = 0.0
    n_group: Optional[int] = None
    topk_group: Optional[int] = None
    devices_per_group: int = 1

    def __post_init__(self):
        if self.expert_num < 1 or self.num_experts_chosen > self.expert_num:
            raise ValueError("expert_num must be >= 1 and num_experts_chosen <= expert_num")
        if self.capacity_factor <= 0:
            raise ValueError("capacity_factor must be positive")


class TopkRouterV2(nn.Module):
    """Returns ``(dispatch [T, k] slot or -1, combine [T, k] weights, expert ids [T, k], aux loss)``."""

    def __init__(self, hidden_size: int, cfg: MoEConfig, device=None):
        super().__init__()
        self.cfg = cfg
        self.gate = nn.Linear(hidden_size, cfg.expert_num, bias=False, device=device, dtype=torch.float32)

    def capacity(self, tokens: int) -> int:
        c = self.cfg
        return max(1, math.ceil(c.capacity_factor * tokens * c.num_experts_chosen / c.expert_num))

    def forward(self, x: torch.Tensor):
        c = self.cfg
        T, E, k = x.shape[0], c.expert_num, c.num_experts_chosen
        logits = self.gate(x.float())
        probs = torch.softmax(logits, dim=-1)
        top_p, top_e = probs.topk(k, dim=-1)
        if c.norm_topk_prob and k > 1:
            top_p = top_p / (top_p.sum(-1, keepdim=True) + 1e-9)
        top_p = top_p * c.routed_scaling_factor
        cap = self.capacity(T)
        onehot = F.one_hot(top_e, E)                                   # [T, k, E]
        if c.enable_sdrop:
            # s-drop: order all T*k copies of an expert by token first (sequence order decides who is dropped)
            flat = onehot.reshape(T * k, E)
            pos = (flat.cumsum(0) - flat).reshape(T, k, E)
        else:
            # k-drop: first choices of all tokens are placed before any second choice
            per_choice = onehot.permute(1, 0, 2).reshape(k * T, E)
            pos = (per_choice.cumsum(0) - per_choice).reshape(k, T, E).permute(1, 0, 2)
        slot = (pos * onehot).sum(-1)                                   # position of the copy inside its expert
        keep = slot < cap
        dispatch = torch.where(keep, slot, torch.full_like(slot, -1))
        combine = top_p * keep
        aux = x.new_zeros((), dtype=torch.float32)
        frac = onehot.sum(1).float().mean(0) / k if k else onehot.float().mean((0, 1))      # f_i
        mean_p = probs.mean(0)                                                                 # P_i
        for kind, factor in zip(c.aux_loss_types, c.aux_loss_factors):
            if kind == "expert":
                aux = aux + factor * E * torch.sum(frac.detach() * mean_p)
            elif kind in ("device", "comm"):
                g = max(1, c.devices_per_group)
                D = E // g
                fd, pd = frac.view(D, g).sum(-1), mean_p.view(D, g).sum(-1)
                aux = aux + factor * D * torch.sum(fd.detach() * pd)
        if c.z_loss_factor:
            aux = aux + c.z_loss_factor * torch.logsumexp(logits, -1).pow(2).mean()
        self.last_drop_rate = 1.0 - keep.float().mean()
        return dispatch, combine, top_e, aux


class MoEV2(nn.Module):
    """Router + batched experts ``[E, capacity, H]`` (+ shared experts)."""

    def __init__(self, hidden_size: int, ffn_hidden_size: int, cfg: MoEConfig, device=None, dtype=torch.float32):
        super().__init__()
        self.cfg, self.H = cfg, hidden_size
        F_ = cfg.moe_intermediate_size or ffn_hidden_size
        E = cfg.expert_num
        self.router = TopkRouterV2(hidden_size, cfg, device)
        self.w1 = nn.Parameter(torch.empty(E, hidden_size, 2 * F_, device=device, dtype=dtype).normal_(0, 0.02))
        self.w2 = nn.Parameter(torch.empty(E, F_, hidden_size, device=device, dtype=dtype).normal_(0, 0.02))
        if cfg.shared_expert_num:
            Fs = F_ * cfg.shared_expert_num
            self.shared_fc1 = nn.Linear(hidden_size, 2 * Fs, bias=False, device=device, dtype=dtype)
            self.shared_fc2 = nn.Linear(Fs, hidden_size, bias=False, device=device, dtype=dtype)
            self.shared_gate = nn.Linear(hidden_size, 1, bias=False, device=device, dtype=dtype) if cfg.use_shared_expert_gating else None
        else:
            self.shared_fc1 = None

    def forward(self, x: torch.Tensor):
        shape = x.shape
        x2 = x.reshape(-1, self.H)
        T, E = x2.shape[0], self.cfg.expert_num
        dispatch, combine, top_e, aux = self.router(x2)
        cap = self.router.capacity(T)
        buf = x2.new_zeros(E * cap + 1, self.H)                         # last row swallows dropped copies
        flat_slot = torch.where(dispatch >= 0, top_e * cap + dispatch, torch.full_like(dispatch, E * cap))
        src = x2.unsqueeze(1).expand(-1, dispatch.shape[1], -1).reshape(-1, self.H)
        buf = buf.index_copy(0, flat_slot.reshape(-1), src)
        h = torch.bmm(buf[:-1].view(E, cap, self.H), self.w1.to(x2.dtype))
        g, u = h.chunk(2, dim=-1)
        y = torch.bmm(F.silu(g) * u, self.w2.to(x2.dtype)).reshape(E * cap, self.H)
        y = torch.cat([y, y.new_zeros(1, self.H)])
        out = (y.index_select(0, flat_slot.reshape(-1)).view(T, -1, self.H) * combine.unsqueeze(-1).to(y.dtype)).sum(1)
        if self.shared_fc1 is not None:
            g, u = self.shared_fc1(x2).chunk(2, dim=-1)
            s = self.shared_fc2(F.silu(g) * u)
            if self.shared_gate is not None:
                s = s * torch.sigmoid(self.shared_gate(x2))
            out = out + s
        return out.reshape(shape), aux


class MoEV3(nn.Module):
    """Dropless MoE with explicit collectives (reference ``modules/transformer/moev3.py:57``, ``ffn_forward_func``
    :491-530): all-to-all of the per-expert counts, all-to-all-v of the token copies sorted by expert, grouped expert
    MLP on the received rows, all-to-all-v back, weighted un-permute. ``group`` is the expert-parallel process group
    (None = all experts local); every rank owns ``expert_num / group size`` consecutive experts.

    The reference's hierarchical variant (inter-node all-gather + intra-node all-to-all-v, ``:689-752``) is a topology
    optimisation for several nodes; on one NVSwitch box every peer is equally far and the flat exchange is used."""

    def __init__(self, hidden_size: int, ffn_hidden_size: int, cfg: MoEConfig, group=None, device=None,
                 dtype=torch.float32):
        super().__init__()
        import torch.distributed as dist
        self.cfg, self.H, self.group = cfg, hidden_size, group
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        if cfg.expert_num % self.world:
            raise ValueError("expert_num must be divisible by the expert-parallel size")
        self.E_local = cfg.expert_num // self.world
        F_ = cfg.moe_intermediate_size or ffn_hidden_size
        self.gate = nn.Linear(hidden_size, cfg.expert_num, bias=False, device=device, dtype=torch.float32)
        g = torch.Generator().manual_seed(4321)                       # full stacks first: values independent of ep
        w1 = torch.empty(cfg.expert_num, hidden_size, 2 * F_).normal_(0, 0.02, generator=g)
        w2 = torch.empty(cfg.expert_num, F_, hidden_size).normal_(0, 0.02, generator=g)
        lo = self.rank * self.E_local
        self.w1 = nn.Parameter(w1[lo:lo + self.E_local].to(device=device, dtype=dtype))
        self.w2 = nn.Parameter(w2[lo:lo + self.E_local].to(device=device, dtype=dtype))

    def route(self, x2: torch.Tensor):
        c = self.cfg
        logits = self.gate(x2.float())
        probs = torch.softmax(logits, dim=-1)
        top_p, top_e = probs.topk(c.num_experts_chosen, dim=-1)
        if c.norm_topk_prob and c.num_experts_chosen > 1:
            top_p = top_p / (top_p.sum(-1, keepdim=True) + 1e-9)
        frac = F.one_hot(top_e, c.expert_num).sum(1).float().mean(0) / c.num_experts_chosen
        aux = c.aux_loss_factor * c.expert_num * torch.sum(frac.detach() * probs.mean(0))
        return top_p * c.routed_scaling_factor, top_e, aux

    def experts(self, rows: torch.Tensor, counts_per_local_expert: torch.Tensor) -> torch.Tensor:
        out = torch.empty_like(rows)
        start = 0
        for e, n in enumerate(counts_per_local_expert.tolist()):
            if n:
                seg = rows[start:start + n]
                g, u = (seg @ self.w1[e].to(seg.dtype)).chunk(2, dim=-1)
                out[start:start + n] = (F.silu(g) * u) @ self.w2[e].to(seg.dtype)
                start += n
        return out

    def forward(self, x: torch.Tensor):
        import torch.distributed as dist
        from ..parallel.mappings import all_to_all
        shape = x.shape
        x2 = x.reshape(-1, self.H)
        T, k, E = x2.shape[0], self.cfg.num_experts_chosen, self.cfg.expert_num
        probs, ids, aux = self.route(x2)
        flat_e = ids.reshape(-1)
        order = torch.argsort(flat_e, stable=True)                    # copies sorted by (global) expert
        send = x2.repeat_interleave(k, dim=0)[order]
        counts = torch.bincount(flat_e, minlength=E)
        if self.world > 1:
            recv_counts = torch.empty_like(counts)
            dist.all_to_all_single(recv_counts, counts, group=self.group)              # counts[r*E_local + e] -> rank r
            in_splits = counts.view(self.world, self.E_local).sum(1).tolist()
            out_splits = recv_counts.view(self.world, self.E_local).sum(1).tolist()
            recv = all_to_all(send, out_splits, in_splits, self.group)               # differentiable exchange
            # received rows are ordered (source rank, local expert): regroup by local expert
            src_counts = recv_counts.view(self.world, self.E_local)
            tag = torch.repeat_interleave(torch.arange(self.E_local, device=x.device).repeat(self.world), src_counts.reshape(-1))
            regroup = torch.argsort(tag, stable=True)
            y = self.experts(recv[regroup], src_counts.sum(0))
            back = torch.zeros_like(y).index_copy(0, regroup, y)
            ret = all_to_all(back, in_splits, out_splits, self.group)
        else:
            ret = self.experts(send, counts)
        unsorted = torch.zeros_like(ret).index_copy(0, order, ret)
        out = (unsorted.view(T, k, self.H) * probs.unsqueeze(-1).to(ret.dtype)).sum(1)
        return out.reshape(shape), aux


class MoEInfer(MoEV3):
    """Forward-only MoE of the legacy inference path (``modules/transformer/moe.py:1888``): routing, expert MLPs and
    the final weighted un-permute (``MoeFinalizeRouting``) without an auxiliary loss."""

    @torch.no_grad()
    def forward(self, x: torch.Tensor):
        out, _ = super().forward(x)
        return out
