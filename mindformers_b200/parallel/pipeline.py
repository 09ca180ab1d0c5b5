"""Pipeline-parallel schedules: 1F1B and interleaved (virtual stages) 1F1B over NCCL point-to-point.

The reference tags layers with ``pipeline_stage`` and lets MindSpore's ``PipelineCell`` schedule micro-batches and
insert Send/Recv (``trainer/base_trainer.py:506-518``, ``training_graph/transformer/utils.py:129-146``); loss is
valid on the last stage only and the token-count denominator is all-reduced over the pipeline group
(``wrapper/wrapper.py:574,607``). Here the schedule is explicit and is data: ``build_schedule`` returns, for one
rank, the list of steps (which virtual micro-batch runs forward, which runs backward, what is sent and received
after each), and ``run_schedule`` executes it. The same lists feed a blocking-rendezvous simulation in the tests,
which shows for every rank count and chunk count that no rank waits on a message whose sender waits on it.

Communication layout, chosen so that the order of operations cannot deadlock:

* activations travel on one communicator, gradients on another (two process groups over the same ranks, so each has
  its own NCCL stream): a blocked activation send never sits in front of a gradient receive;
* on each communicator a step issues ONE ``batch_isend_irecv`` that holds the send of what the step produced and the
  receive of what the rank needs next. Both run concurrently inside the batch, so the wrap-around traffic of the
  interleaved schedule (last stage -> first stage, next chunk) cannot form a cycle of sends that wait for receives
  queued behind other sends;
* the activation batch is issued right after the forward and awaited before the next forward, the gradient batch
  right after the backward and awaited before the next backward: the transfers overlap the other half of the step;
* receive buffers are allocated on the compute stream at issue time and the communicator's stream orders itself
  after that stream, so a recycled block is never written while earlier kernels still read it.

Schedules: warm-up forwards (``pp - rank - 1``; with ``v`` chunks per rank ``2 (pp - rank - 1) + (v - 1) pp``), then
one-forward-one-backward, then cool-down backwards. Virtual micro-batch ``k`` runs chunk ``(k // pp) % v`` forward and
chunk ``v - 1 - (k // pp) % v`` backward, which divides the bubble by ``v``. The embedding weight shared by the first
and the last stage gets its gradient all-reduced over those two ranks.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from . import parallel_state as ps

_EMBED_GROUPS: Dict[tuple, object] = {}


@dataclass
class Step:
    """One entry of a rank's schedule. ``fwd`` / ``bwd``: virtual micro-batch to run forward / backward (``None``: none).
    After the forward the activation batch goes out: ``send_act`` (output of that forward to the next stage) and
    ``recv_act`` (input of virtual micro-batch ``recv_act`` from the previous stage). After the backward the gradient
    batch: ``send_grad`` (input gradient to the previous stage), ``recv_grad`` (output gradient of ``recv_grad``)."""

    fwd: Optional[int] = None
    bwd: Optional[int] = None
    send_act: Optional[int] = None
    recv_act: Optional[int] = None
    send_grad: Optional[int] = None
    recv_grad: Optional[int] = None


def fwd_chunk(k: int, pp: int, v: int) -> int:
    return (k // pp) % v


def bwd_chunk(k: int, pp: int, v: int) -> int:
    return v - 1 - (k // pp) % v


def microbatch_of(k: int, pp: int, v: int) -> int:
    return (k // (pp * v)) * pp + k % pp


def build_schedule(pp: int, v: int, n: int, rank: int) -> List[Step]:
    """Steps of ``rank`` for ``n`` micro-batches over ``pp`` stages with ``v`` model chunks per rank."""
    if v > 1 and n % pp != 0:
        raise ValueError(f"interleaved schedule needs micro-batches ({n}) to be a multiple of pipeline stages ({pp})")
    total = n * v
    warm = min((pp - rank - 1) * (2 if v > 1 else 1) + (v - 1) * pp, total)

    def needs_act(k):          # the first chunk of the first stage embeds its own input
        return 0 <= k < total and not (rank == 0 and fwd_chunk(k, pp, v) == 0)

    def sends_act(k):          # the last chunk of the last stage produces the loss
        return not (rank == pp - 1 and fwd_chunk(k, pp, v) == v - 1)

    def needs_grad(k):
        return 0 <= k < total and not (rank == pp - 1 and bwd_chunk(k, pp, v) == v - 1)

    def sends_grad(k):
        return not (rank == 0 and bwd_chunk(k, pp, v) == 0)

    steps = [Step(recv_act=0 if needs_act(0) else None, recv_grad=0 if (warm == 0 and needs_grad(0)) else None)]
    for k in range(warm):
        st = Step(fwd=k, send_act=k if sends_act(k) else None, recv_act=k + 1 if needs_act(k + 1) else None)
        if k == warm - 1 and needs_grad(0):
            st.recv_grad = 0
        steps.append(st)
    for i in range(total - warm):
        f, b = warm + i, i
        steps.append(Step(fwd=f, bwd=b, send_act=f if sends_act(f) else None,
                          recv_act=f + 1 if needs_act(f + 1) else None,
                          send_grad=b if sends_grad(b) else None, recv_grad=b + 1 if needs_grad(b + 1) else None))
    for b in range(total - warm, total):
        steps.append(Step(bwd=b, send_grad=b if sends_grad(b) else None, recv_grad=b + 1 if needs_grad(b + 1) else None))
    return steps


class P2PCommunicator:
    """Activation and gradient exchange with the neighbouring stages: one batched send+receive per ring per step."""

    def __init__(self, shape: Sequence[int], dtype: torch.dtype, device):
        self.shape, self.dtype, self.device = tuple(shape), dtype, torch.device(device)
        self.act_group = ps.get_pipeline_model_parallel_group()
        self.grad_group = backward_group()
        self.pp = ps.get_pipeline_model_parallel_world_size()
        self.next = ps.get_pipeline_model_parallel_next_rank() if self.pp > 1 else None
        self.prev = ps.get_pipeline_model_parallel_prev_rank() if self.pp > 1 else None
        self.bytes_sent = 0

    def _batch(self, send: Optional[torch.Tensor], dst, recv: bool, src, group):
        """Issue one batch holding at most one send and one receive; returns (receive buffer or None, requests, the
        tensors that must stay alive until the requests were awaited)."""
        ops, keep, buf = [], [], None
        if send is not None:
            send = send.contiguous()
            keep.append(send)
            self.bytes_sent += send.numel() * send.element_size()
            ops.append(dist.P2POp(dist.isend, send, dst, group))
        if recv:
            buf = torch.empty(self.shape, dtype=self.dtype, device=self.device)
            ops.append(dist.P2POp(dist.irecv, buf, src, group))
        reqs = dist.batch_isend_irecv(ops) if ops else []
        return buf, reqs, keep

    def exchange_act(self, send: Optional[torch.Tensor], recv: bool):
        return self._batch(None if send is None else send.detach(), self.next, recv, self.prev, self.act_group)

    def exchange_grad(self, send: Optional[torch.Tensor], recv: bool):
        return self._batch(send, self.prev, recv, self.next, self.grad_group)

    @staticmethod
    def wait(pending):
        if pending is None:
            return None
        buf, reqs, _keep = pending
        for r in reqs:
            r.wait()
        return buf


def _forward_step(model, mb, input_tensor, num_microbatches, collect, loss_scale):
    """One micro-batch forward on one model chunk; returns what must be sent on / differentiated."""
    if input_tensor is not None:
        model.set_input_tensor(input_tensor)
    out = model(mb["input_ids"], mb.get("labels"), mb.get("loss_mask"), mb.get("position_ids"))
    aux = None
    if model.post_process:
        loss = out
        collect.append(loss.detach())
        return loss * (loss_scale / num_microbatches), None
    if isinstance(out, tuple):
        out, aux = out
        aux = aux * (loss_scale / num_microbatches)
    return out, aux


def _backward_step(input_tensor, output, aux, output_grad):
    if input_tensor is not None and input_tensor.grad is not None:
        input_tensor.grad = None
    if output_grad is None:        # last stage: output is the scaled loss
        output.backward()
    else:
        tensors, grads = [output], [output_grad]
        if aux is not None:
            tensors.append(aux)
            grads.append(torch.ones_like(aux))
        torch.autograd.backward(tensors, grads)
    return None if input_tensor is None else input_tensor.grad


def forward_backward_no_pipelining(model, microbatches: List[dict], loss_scale: float = 1.0):
    losses: List[torch.Tensor] = []
    n = len(microbatches)
    for mb in microbatches:
        out, _ = _forward_step(model, mb, None, n, losses, loss_scale)
        out.backward()
    return losses


def run_schedule(chunks: List[torch.nn.Module], microbatches: List[dict], hidden_shape, dtype,
                 loss_scale: float = 1.0) -> List[torch.Tensor]:
    """Execute this rank's schedule (``build_schedule``) over its model chunks; returns the micro-batch losses on
    the rank that holds the last chunk of the last stage."""
    pp = ps.get_pipeline_model_parallel_world_size()
    rank = ps.get_pipeline_model_parallel_rank()
    v, n = len(chunks), len(microbatches)
    steps = build_schedule(pp, v, n, rank)
    dev = next(chunks[0].parameters()).device
    comm = P2PCommunicator(hidden_shape, dtype, dev)
    losses: List[torch.Tensor] = []
    inputs = [[] for _ in range(v)]
    outputs = [[] for _ in range(v)]
    auxes = [[] for _ in range(v)]
    act_pending = grad_pending = None       # the batch in flight on each ring
    act_in: Dict[int, torch.Tensor] = {}    # received inputs / output gradients by virtual micro-batch
    grad_in: Dict[int, torch.Tensor] = {}

    def finish_act(st_prev):
        nonlocal act_pending
        buf = comm.wait(act_pending)
        act_pending = None
        if buf is not None:
            act_in[st_prev.recv_act] = buf.requires_grad_()

    def finish_grad(st_prev):
        nonlocal grad_pending
        buf = comm.wait(grad_pending)
        grad_pending = None
        if buf is not None:
            grad_in[st_prev.recv_grad] = buf

    act_owner = grad_owner = None           # the step whose batch is in flight
    for st in steps:
        y = gx = None
        if st.fwd is not None:
            if act_owner is not None:
                finish_act(act_owner)
                act_owner = None
            k = st.fwd
            c = fwd_chunk(k, pp, v)
            if v > 1:
                ps.set_virtual_pipeline_model_parallel_rank(c)
            x = act_in.pop(k, None)
            y, aux = _forward_step(chunks[c], microbatches[microbatch_of(k, pp, v)], x, n, losses, loss_scale)
            inputs[c].append(x); outputs[c].append(y); auxes[c].append(aux)
        if st.send_act is not None or st.recv_act is not None:
            if act_owner is not None:       # a batch of a step without a forward (the first receive) is still in flight
                finish_act(act_owner)
            act_pending = comm.exchange_act(y if st.send_act is not None else None, st.recv_act is not None)
            act_owner = st
        if st.bwd is not None:
            if grad_owner is not None:
                finish_grad(grad_owner)
                grad_owner = None
            k = st.bwd
            c = bwd_chunk(k, pp, v)
            if v > 1:
                ps.set_virtual_pipeline_model_parallel_rank(c)
            g = grad_in.pop(k, None)
            xi, yo, au = inputs[c].pop(0), outputs[c].pop(0), auxes[c].pop(0)
            gx = _backward_step(xi, yo, au, g)
        if st.send_grad is not None or st.recv_grad is not None:
            if grad_owner is not None:
                finish_grad(grad_owner)
            grad_pending = comm.exchange_grad(gx if st.send_grad is not None else None, st.recv_grad is not None)
            grad_owner = st
    if act_owner is not None:
        finish_act(act_owner)
    if grad_owner is not None:
        finish_grad(grad_owner)
    if v > 1:
        ps.set_virtual_pipeline_model_parallel_rank(0)
    run_schedule.last_bytes_sent = comm.bytes_sent
    return losses


def forward_backward_pipelining_without_interleaving(model, microbatches: List[dict], hidden_shape, dtype,
                                                     loss_scale: float = 1.0, overlap: bool = True):
    """Non-interleaved 1F1B. ``model`` is this stage's chunk; returns the micro-batch losses on the last stage."""
    return run_schedule([model], microbatches, hidden_shape, dtype, loss_scale)


def forward_backward_pipelining_with_interleaving(chunks: List[torch.nn.Module], microbatches: List[dict], hidden_shape,
                                                  dtype, loss_scale: float = 1.0, overlap: bool = True):
    """Interleaved 1F1B over ``v = len(chunks)`` model chunks per rank. The number of micro-batches must be a
    multiple of the pipeline size."""
    return run_schedule(list(chunks), microbatches, hidden_shape, dtype, loss_scale)


def get_forward_backward_func():
    pp = ps.get_pipeline_model_parallel_world_size()
    if pp == 1:
        return forward_backward_no_pipelining
    if (ps.get_virtual_pipeline_model_parallel_world_size() or 1) > 1:
        return forward_backward_pipelining_with_interleaving
    return forward_backward_pipelining_without_interleaving


# ----------------------------------------------------------------------------------------------------
def _build_side_groups():
    """Collective (whole job): for every pipeline group, a second communicator for gradients and the
    (first stage, last stage) pair for the tied embedding."""
    world = dist.get_world_size()
    if ("built", world) in _EMBED_GROUPS:
        return
    pp_ranks = tuple(ps.get_group_ranks("pp"))
    all_pp = [None] * world
    dist.all_gather_object(all_pp, pp_ranks)
    seen = []
    for ranks in all_pp:
        if ranks not in seen:
            seen.append(ranks)
    for ranks in seen:
        pair = sorted({ranks[0], ranks[-1]})
        _EMBED_GROUPS[ranks] = dist.new_group(ranks=pair) if len(pair) > 1 else None
        _EMBED_GROUPS[("bwd",) + ranks] = dist.new_group(ranks=list(ranks)) if len(ranks) > 1 else None
    _EMBED_GROUPS[("built", world)] = True


def backward_group():
    if ps.get_pipeline_model_parallel_world_size() == 1 or not dist.is_initialized():
        return None
    _build_side_groups()
    return _EMBED_GROUPS.get(("bwd",) + tuple(ps.get_group_ranks("pp")))


def embedding_group():
    """Process group of the first and last pipeline stage of this rank's pipeline (created collectively)."""
    _build_side_groups()
    pp_ranks = tuple(ps.get_group_ranks("pp"))
    return _EMBED_GROUPS.get(pp_ranks)


def sync_shared_embedding_grads(chunks: Sequence[torch.nn.Module]):
    """All-reduce the gradient of the tied embedding / output weight between the first and the last stage."""
    pp = ps.get_pipeline_model_parallel_world_size()
    if pp == 1:
        return
    grp = embedding_group()
    rank = ps.get_pipeline_model_parallel_rank()
    if rank not in (0, pp - 1) or grp is None:
        return
    model = chunks[0] if rank == 0 else chunks[-1]
    if not getattr(model, "tied", False):
        return
    w = model.shared_embedding_or_output_weight()
    g = getattr(w, "main_grad", None)
    if g is None:
        g = w.grad
    if g is not None:
        dist.all_reduce(g, group=grp)


class PipelineTrainStep:
    """Train step for ``pp > 1``: splits the rank's batch into micro-batches, runs the schedule, reduces and steps.

    ``chunks``: the model chunks of this rank (one unless virtual stages are used); ``optimizer`` covers all of them.
    Returns the same dictionary as ``TrainOneStep``; the loss is broadcast from the last stage.
    """

    def __init__(self, chunks: Sequence[torch.nn.Module], optimizer, micro_batch_size: int = 1, loss_scale: float = 1.0,
                 overlap: bool = True):
        self.chunks = list(chunks)
        self.optimizer, self.mbs, self.loss_scale, self.overlap = optimizer, micro_batch_size, loss_scale, overlap

    def __call__(self, batch: Dict[str, torch.Tensor]):
        cfg = self.chunks[0].config
        n = batch["input_ids"].shape[0] // self.mbs
        mbs = [{k: v[i * self.mbs:(i + 1) * self.mbs] for k, v in batch.items() if v is not None} for i in range(n)]
        S = batch["input_ids"].shape[1]
        tp = ps.get_tensor_model_parallel_world_size()
        T = self.mbs * S // (tp if cfg.sequence_parallel else 1)
        shape = (T, cfg.hidden_size)
        dtype = cfg.compute_dtype if isinstance(cfg.compute_dtype, torch.dtype) else getattr(torch, str(cfg.compute_dtype))
        self.optimizer.zero_grad()
        if len(self.chunks) > 1:
            losses = forward_backward_pipelining_with_interleaving(self.chunks, mbs, shape, dtype, self.loss_scale, self.overlap)
        elif ps.get_pipeline_model_parallel_world_size() > 1:
            losses = forward_backward_pipelining_without_interleaving(self.chunks[0], mbs, shape, dtype, self.loss_scale,
                                                                     self.overlap)
        else:
            losses = forward_backward_no_pipelining(self.chunks[0], mbs, self.loss_scale)
        sync_shared_embedding_grads(self.chunks)
        dp = ps.get_data_parallel_world_size(with_context_parallel=True)
        scale = 1.0 / (dp * self.loss_scale)
        self.optimizer.step(grad_scale=scale)
        dev = batch["input_ids"].device
        loss = torch.stack(losses).mean() if losses else torch.zeros((), device=dev)
        pp_group = ps.get_pipeline_model_parallel_group()
        if pp_group is not None and ps.get_pipeline_model_parallel_world_size() > 1:
            loss = loss.clone().float()
            last_global = ps.get_group_ranks("pp")[-1]
            dist.broadcast(loss, src=last_global, group=pp_group)
        return {"loss": loss, "global_norm": self.optimizer.global_norm(scale), "skipped": self.optimizer.skipped,
                "lr": self.optimizer.current_lr(), "loss_scale": self.loss_scale}
