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
