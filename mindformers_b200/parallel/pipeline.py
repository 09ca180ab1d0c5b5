"""Pipeline-parallel schedules: 1F1B and interleaved (virtual stages) 1F1B over NCCL point-to-point.

The reference tags layers with ``pipeline_stage`` and lets MindSpore's ``PipelineCell`` schedule micro-batches and
insert Send/Recv (``trainer/base_trainer.py:506-518``, ``training_graph/transformer/utils.py:129-146``); loss is
valid on the last stage only and the token-count denominator is all-reduced over the pipeline group
(``wrapper/wrapper.py:574,607``). Here the schedule is explicit:

* activations ``[T, H]`` travel with ``torch.distributed.batch_isend_irecv``; on CUDA the transfers are issued
  from a side stream that waits on the producing kernel through an event, so the next micro-batch's compute on the
  main stream overlaps the transfer; a receive is posted one step ahead of its use;
* warm-up forwards (``pp - rank - 1``), steady one-forward-one-backward, cool-down backwards;
* with ``virtual_pipeline_model_parallel_size = v`` every rank owns ``v`` model chunks and micro-batches visit
  chunk ``c`` of all stages before chunk ``c + 1`` (interleaved 1F1B), which divides the bubble by ``v``;
* the embedding weight shared by the first and the last stage gets its gradient all-reduced over those two ranks.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from . import parallel_state as ps

_EMBED_GROUPS: Dict[tuple, object] = {}


class P2PCommunicator:
    """Send/receive of activations and their gradients to the neighbouring stages."""

    def __init__(self, shape: Sequence[int], dtype: torch.dtype, device, overlap: bool = True):
        self.shape, self.dtype, self.device = tuple(shape), dtype, torch.device(device)
        # activations and gradients travel on separate communicators: between one pair of ranks each then carries a
        # single kind of message, whose order is the micro-batch order on both sides (with two stages and virtual
        # chunks, wrap-around gradients and ordinary activations would otherwise share a queue)
        self.group = ps.get_pipeline_model_parallel_group()
        self.bwd_group = backward_group()
        self.pp = ps.get_pipeline_model_parallel_world_size()
        self.rank = ps.get_pipeline_model_parallel_rank()
        self.next = ps.get_pipeline_model_parallel_next_rank() if self.pp > 1 else None
        self.prev = ps.get_pipeline_model_parallel_prev_rank() if self.pp > 1 else None
        self.cuda = self.device.type == "cuda"
        self.stream = torch.cuda.Stream(device=self.device) if (self.cuda and overlap) else None
        self.bytes_sent = 0
        self._keep: List[torch.Tensor] = []

    def _issue(self, ops, produced: Optional[torch.Tensor] = None):
        if not ops:
            return []
        if self.stream is not None:
            if produced is not None:
                self.stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.stream):
                reqs = dist.batch_isend_irecv(ops)
            return reqs
        return dist.batch_isend_irecv(ops)

    def _wait(self, reqs):
        for r in reqs:
            r.wait()
        if self.stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.stream)

    def irecv(self, src, group) -> tuple:
        buf = torch.empty(self.shape, dtype=self.dtype, device=self.device)
        if self.stream is not None:
            buf.record_stream(self.stream)
        reqs = self._issue([dist.P2POp(dist.irecv, buf, src, group)])
        return buf, reqs

    def isend(self, t: torch.Tensor, dst, group):
        t = t.contiguous()
        if self.stream is not None:
            t.record_stream(self.stream)
        self._keep.append(t)
        if len(self._keep) > 4 * max(self.pp, 2):
            self._keep = self._keep[-2 * max(self.pp, 2):]
        self.bytes_sent += t.numel() * t.element_size()
        return self._issue([dist.P2POp(dist.isend, t, dst, group)], produced=t)

    # blocking forms used by the schedules ------------------------------------------------------------
    def recv_forward(self, first: bool):
        if first:
            return None
        buf, reqs = self.irecv(self.prev, self.group)
        self._wait(reqs)
        return buf.requires_grad_()

    def recv_backward(self, last: bool):
        if last:
            return None
        buf, reqs = self.irecv(self.next, self.bwd_group)
        self._wait(reqs)
        return buf

    def send_forward(self, t, last: bool):
        if not last:
            self._pending = getattr(self, "_pending", []) + self.isend(t.detach(), self.next, self.group)

    def send_backward(self, g, first: bool):
        if not first:
            self._pending = getattr(self, "_pending", []) + self.isend(g, self.prev, self.bwd_group)

    def flush(self):
        for r in getattr(self, "_pending", []):
            r.wait()
        self._pending = []
        if self.stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.stream)


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


def forward_backward_pipelining_without_interleaving(model, microbatches: List[dict], hidden_shape, dtype,
                                                     loss_scale: float = 1.0, overlap: bool = True):
    """Non-interleaved 1F1B. ``model`` is this stage's chunk; returns the micro-batch losses on the last stage."""
    pp = ps.get_pipeline_model_parallel_world_size()
    rank = ps.get_pipeline_model_parallel_rank()
    first, last = rank == 0, rank == pp - 1
    n = len(microbatches)
    dev = next(model.parameters()).device
    comm = P2PCommunicator(hidden_shape, dtype, dev, overlap)
    warm = min(pp - rank - 1, n)
    steady = n - warm
    losses: List[torch.Tensor] = []
    inputs, outputs, auxes = [], [], []
    k = 0
    for _ in range(warm):
        x = comm.recv_forward(first)
        y, aux = _forward_step(model, microbatches[k], x, n, losses, loss_scale)
        comm.send_forward(y, last)
        inputs.append(x); outputs.append(y); auxes.append(aux)
        k += 1
    x = comm.recv_forward(first) if steady > 0 else None
    for i in range(steady):
        y, aux = _forward_step(model, microbatches[k], x, n, losses, loss_scale)
        k += 1
        comm.send_forward(y, last)
        inputs.append(x); outputs.append(y); auxes.append(aux)
        g = comm.recv_backward(last)
        xi, yo, au = inputs.pop(0), outputs.pop(0), auxes.pop(0)
        gx = _backward_step(xi, yo, au, g)
        comm.send_backward(gx, first)
        if i < steady - 1:
            x = comm.recv_forward(first)
    for _ in range(warm):
        g = comm.recv_backward(last)
        xi, yo, au = inputs.pop(0), outputs.pop(0), auxes.pop(0)
        gx = _backward_step(xi, yo, au, g)
        comm.send_backward(gx, first)
    comm.flush()
    return losses


def forward_backward_pipelining_with_interleaving(chunks: List[torch.nn.Module], microbatches: List[dict], hidden_shape,
                                                  dtype, loss_scale: float = 1.0, overlap: bool = True):
    """Interleaved 1F1B over ``v = len(chunks)`` model chunks per rank. The number of micro-batches must be a
    multiple of the pipeline size. Virtual micro-batch ``j`` runs chunk ``(j // pp) % v`` (forward order); the
    backward order mirrors it from the last chunk."""
    pp = ps.get_pipeline_model_parallel_world_size()
    rank = ps.get_pipeline_model_parallel_rank()
    v = len(chunks)
    n = len(microbatches)
    if n % pp != 0:
        raise ValueError(f"interleaved schedule needs micro-batches ({n}) to be a multiple of pipeline stages ({pp})")
    total = n * v
    dev = next(chunks[0].parameters()).device
    comm = P2PCommunicator(hidden_shape, dtype, dev, overlap)
    losses: List[torch.Tensor] = []

    def chunk_of(j, forward=True):
        c = (j // pp) % v
        return c if forward else v - 1 - c

    def mb_of(j):
        return (j // (pp * v)) * pp + j % pp

    warm = min((pp - rank - 1) * 2 + (v - 1) * pp, total)
    steady = total - warm
    inputs = [[] for _ in range(v)]
    outputs = [[] for _ in range(v)]
    auxes = [[] for _ in range(v)]

    def is_first(c):
        return rank == 0 and c == 0

    def is_last(c):
        return rank == pp - 1 and c == v - 1

    def fwd(j):
        c = chunk_of(j)
        ps.set_virtual_pipeline_model_parallel_rank(c)
        x = comm.recv_forward(is_first(c))
        y, aux = _forward_step(chunks[c], microbatches[mb_of(j)], x, n, losses, loss_scale)
        comm.send_forward(y, is_last(c))
        inputs[c].append(x); outputs[c].append(y); auxes[c].append(aux)

    def bwd(j):
        c = chunk_of(j, forward=False)
        ps.set_virtual_pipeline_model_parallel_rank(c)
        g = comm.recv_backward(is_last(c))
        xi, yo, au = inputs[c].pop(0), outputs[c].pop(0), auxes[c].pop(0)
        gx = _backward_step(xi, yo, au, g)
        comm.send_backward(gx, is_first(c))

    for j in range(warm):
        fwd(j)
    for i in range(steady):
        fwd(warm + i)
        bwd(i)
    for i in range(steady, total):
        bwd(i)
    comm.flush()
    ps.set_virtual_pipeline_model_parallel_rank(0)
    return losses


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
