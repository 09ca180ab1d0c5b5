"""Token dispatchers of the mixture-of-experts layer beyond the plain all-to-all one.

``StagedTokenDispatcher`` moves the ``T·k`` token copies of a rank to the experts that were chosen for them and
brings the expert outputs back, as a sequence of stages that can be combined:

* ``kind="alltoall"`` — copies sorted by expert, one all-to-all-v over the expert-parallel group
  (reference ``training_graph/transformer/moe/token_dispatcher.py:94-270``).
* ``kind="allgather"`` — tokens, routing and weights are all-gathered over the expert-parallel group, every rank keeps
  the copies of its own experts, outputs are weighted, scattered back onto a token-indexed buffer and
  reduce-scattered (the dispatcher the reference's inference MoE and Megatron call all-gather).
* ``kind="deredundency"`` — the two-level form of the legacy stack (``modules/transformer/moev3.py:395-456,647-756``,
  ``enable_deredundency`` / ``npu_nums_per_device``): ranks are grouped into nodes of ``inner`` ranks; tokens are
  all-gathered across nodes only (between the ranks with the same position in their node), so a token crosses the
  inter-node link once however many experts of that node it was routed to; inside the node an all-to-all-v takes each
  copy to the rank that holds its expert; the way back ends in a reduce-scatter across nodes.
* expert tensor parallelism (``etp > 1``, ``moev3.py:758-850`` and Megatron's AG(TP)/RS(TP) around the experts): every
  expert's FFN is sharded over the tensor-parallel ranks, so the rows that the ranks of that group received are
  all-gathered (ragged) before the experts and the partial outputs reduce-scattered (ragged) after.
* safe tokens (``use_pad_tokens`` / ``enable_gmm_safe_tokens``, ``token_dispatcher.py:161-178``, ``moev3.py:1037-1098``):
  one zero row per expert is added so that no expert of any rank sees an empty batch, and removed on the way back.

All stages are differentiable (their backward passes are the mirrored collectives). Split sizes cross to the host
once per layer call, as in the reference (``preprocess`` → ``d2h``).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .. import mappings as M
from .. import parallel_state as ps


# ---------------------------------------------------------------------------------------------------------------
# differentiable collectives over an arbitrary group
# ---------------------------------------------------------------------------------------------------------------
def _size(group) -> int:
    return dist.get_world_size(group) if group is not None else 1


class _AllGatherRows(torch.autograd.Function):
    """Concatenate equally sized row blocks of all members; backward: reduce-scatter of the gradient."""
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return M.all_gather_first_dim(x, group, _size(group))

    @staticmethod
    def backward(ctx, g):
        return M.reduce_scatter_first_dim(g, ctx.group, _size(ctx.group)), None


class _ReduceScatterRows(torch.autograd.Function):
    """Sum over the members and keep this member's row block; backward: all-gather of the gradient."""
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return M.reduce_scatter_first_dim(x, group, _size(group))

    @staticmethod
    def backward(ctx, g):
        return M.all_gather_first_dim(g, ctx.group, _size(ctx.group)), None


def _pad_rows(x, n):
    if x.shape[0] == n:
        return x
    return torch.cat((x, x.new_zeros((n - x.shape[0], *x.shape[1:]))), dim=0)


def _gather_ragged(x, counts, group):
    """Row blocks of different lengths (``counts[r]`` rows from member r) → their concatenation."""
    world, big = len(counts), max(max(counts), 1)
    full = M.all_gather_first_dim(_pad_rows(x, big), group, world)
    return torch.cat([full[r * big:r * big + counts[r]] for r in range(world)], dim=0)


def _reduce_scatter_ragged(x, counts, rank, group):
    """Inverse of ``_gather_ragged``: ``x`` holds ``sum(counts)`` rows on every member; sum over the members and return
    the ``counts[rank]`` rows of this one."""
    world, big = len(counts), max(max(counts), 1)
    parts, o = [], 0
    for r in range(world):
        parts.append(_pad_rows(x[o:o + counts[r]], big))
        o += counts[r]
    mine = M.reduce_scatter_first_dim(torch.cat(parts, dim=0), group, world)
    return mine[:counts[rank]]


class _GatherRagged(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, counts, rank, group):
        ctx.meta = (counts, rank, group)
        return _gather_ragged(x, counts, group)

    @staticmethod
    def backward(ctx, g):
        counts, rank, group = ctx.meta
        return _reduce_scatter_ragged(g.contiguous(), counts, rank, group), None, None, None


class _ReduceScatterRagged(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, counts, rank, group):
        ctx.meta = (counts, rank, group)
        return _reduce_scatter_ragged(x, counts, rank, group)

    @staticmethod
    def backward(ctx, g):
        counts, rank, group = ctx.meta
        return _gather_ragged(g.contiguous(), counts, group), None, None, None


def _all_gather_ints(t: torch.Tensor, group) -> torch.Tensor:
    return M.all_gather_first_dim(t.contiguous(), group, _size(group)) if _size(group) > 1 else t


# ---------------------------------------------------------------------------------------------------------------
class StagedTokenDispatcher:
    """See the module docstring. ``dispatch(x [T,H], ids [T,k])`` → ``(expert input in the padded layout, plan, ctx)``;
    ``combine(y, plan, ctx, probs [T,k])`` → ``[T, H]``."""

    KINDS = ("alltoall", "allgather", "deredundency")

    def __init__(self, config, kind: str = "alltoall", inner: Optional[int] = None, expert_tp: bool = False):
        if kind not in self.KINDS:
            raise ValueError(f"moe dispatcher {kind!r}: expected one of {self.KINDS}")
        self.config, self.kind = config, kind
        self.ep = ps.get_expert_model_parallel_world_size()
        self.ep_rank = ps.get_expert_model_parallel_rank()
        self.ep_group = ps.get_expert_model_parallel_group()
        self.E = config.num_moe_experts
        self.E_local = self.E // self.ep
        self.k = config.moe_router_topk
        self.pad = bool(getattr(config, "use_pad_tokens", False))
        self.etp = ps.get_expert_tensor_parallel_world_size() if expert_tp else 1
        self.etp_rank = ps.get_expert_tensor_parallel_rank() if self.etp > 1 else 0
        self.etp_group = ps.get_expert_tensor_parallel_group() if self.etp > 1 else None
        if kind == "allgather":
            inner = 1
        elif kind == "deredundency":
            inner = int(inner or getattr(config, "npu_nums_per_device", 1) or 1)
        else:
            inner = self.ep
        if self.ep % inner:
            raise ValueError(f"expert-parallel size {self.ep} is not a multiple of the inner group size {inner}")
        self.inner = inner
        self.outer = self.ep // inner
        if kind != "alltoall" and self.ep > 1:
            self.inner_group, _, self.outer_group, _ = ps.split_group("ep", inner)
        else:
            self.inner_group, self.outer_group = self.ep_group, None
        self.inner_rank = self.ep_rank % inner
        self.node = self.ep_rank // inner               # experts [node·inner·E_local, (node+1)·inner·E_local) live here

    # ---- stage: all-to-all-v over `group`, copies already sorted by destination ---------------------------------
    def _a2a(self, rows, e_sorted, n_ranks, group):
        """``rows`` sorted by ``e_sorted`` (expert index inside the group's expert range) → rows received by this rank
        with their local expert indices, plus what the way back needs."""
        counts = torch.bincount(e_sorted, minlength=n_ranks * self.E_local).view(n_ranks, self.E_local)
        recv_counts = torch.empty_like(counts)
        dist.all_to_all_single(recv_counts.view(-1), counts.view(-1).contiguous(), group=group)
        in_splits = counts.sum(1).tolist()
        out_splits = recv_counts.sum(1).tolist()
        recv = M.all_to_all(rows, out_splits, in_splits, group)
        local_e = torch.repeat_interleave(torch.arange(self.E_local, device=rows.device).repeat(n_ranks),
                                          recv_counts.view(-1), output_size=recv.shape[0])
        return recv, local_e, (in_splits, out_splits, group)

    # ---- dispatch -------------------------------------------------------------------------------------------------
    def dispatch(self, x, ids):
        from .moe import PermutePlan, permute
        T, H = x.shape
        dev = x.device
        src = torch.arange(T * self.k, device=dev) // self.k
        e = ids.reshape(-1).to(torch.int64)
        Tp = T
        if self.pad:                      # one zero row per expert: token T of the extended input
            src = torch.cat((src, torch.full((self.E,), T, device=dev, dtype=src.dtype)))
            e = torch.cat((e, torch.arange(self.E, device=dev)))
            x = torch.cat((x, x.new_zeros(1, H)), dim=0)
            Tp = T + 1
        ctx = {"T": T, "Tp": Tp, "src": src}
        if self.ep == 1:
            rows, le = x.index_select(0, src), e
        elif self.kind == "alltoall":
            order = torch.argsort(e, stable=True)
            rows, le, ctx["a2a"] = self._a2a(x.index_select(0, src[order]), e[order], self.ep, self.ep_group)
            ctx["inv"] = torch.argsort(order)
        else:
            og = self.outer_group
            xg = _AllGatherRows.apply(x, og) if self.outer > 1 else x
            eg = _all_gather_ints(e, og)
            n_copies = src.shape[0]
            offs = torch.arange(self.outer, device=dev).repeat_interleave(n_copies) * Tp
            srcg = _all_gather_ints(src, og) + offs
            a = self.node * self.inner * self.E_local
            b = a + self.inner * self.E_local
            idx = torch.nonzero((eg >= a) & (eg < b)).reshape(-1)
            sel = idx[torch.argsort(eg[idx], stable=True)]
            rows = xg.index_select(0, srcg[sel])
            le = eg[sel] - a
            ctx.update(sel=sel, srcg=srcg, n_copies=n_copies)
            if self.inner > 1:
                rows, le, ctx["a2a"] = self._a2a(rows, le, self.inner, self.inner_group)
        if self.etp > 1:
            n = torch.tensor([rows.shape[0]], device=dev, dtype=torch.int64)
            counts = _all_gather_ints(n, self.etp_group).tolist()
            rows = _GatherRagged.apply(rows, counts, self.etp_rank, self.etp_group)
            le = _gather_ragged(le, counts, self.etp_group)
            ctx["etp_counts"] = counts
        plan = PermutePlan(le, self.E_local)
        return permute(rows, plan, 1), plan, ctx

    # ---- combine --------------------------------------------------------------------------------------------------
    def combine(self, y, plan, ctx, probs):
        T, Tp, src = ctx["T"], ctx["Tp"], ctx["src"]
        back = y.index_select(0, plan.dest)
        if self.etp > 1:
            back = _ReduceScatterRagged.apply(back, ctx["etp_counts"], self.etp_rank, self.etp_group)
        w = probs.reshape(-1).float()
        if self.pad:
            w = torch.cat((w, w.new_zeros(self.E)))
        if "a2a" in ctx:
            in_splits, out_splits, group = ctx["a2a"]
            back = M.all_to_all(back, in_splits, out_splits, group)
        if self.ep == 1 or self.kind == "alltoall":
            if "inv" in ctx:
                back = back.index_select(0, ctx["inv"])              # copy order again
            out = torch.zeros((Tp, y.shape[1]), dtype=torch.float32, device=y.device)
            out = out.index_add(0, src, back.float() * w.unsqueeze(-1))
        else:
            og, sel = self.outer_group, ctx["sel"]
            wg = _AllGatherRows.apply(w, og) if self.outer > 1 else w
            board = torch.zeros((self.outer * Tp, y.shape[1]), dtype=torch.float32, device=y.device)
            board = board.index_add(0, ctx["srcg"][sel], back.float() * wg[sel].unsqueeze(-1))
            out = _ReduceScatterRows.apply(board, og) if self.outer > 1 else board
        return out[:T].to(y.dtype)
