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


def seq_bwd_unit(b: int, seq_split: int) -> int:
    """Sequence pipeline: the forward unit (micro-batch, chunk) = ``m * C + c`` that the ``b``-th backward handles. The
    chunks of a micro-batch run backward in reverse, because a chunk's keys and values are read by the chunks after
    it and their gradients must be complete first."""
    m, r = divmod(b, seq_split)
    return m * seq_split + (seq_split - 1 - r)


def build_schedule(pp: int, v: int, n: int, rank: int, seq_split: int = 1) -> List[Step]:
    """Steps of ``rank`` for ``n`` micro-batches over ``pp`` stages with ``v`` model chunks per rank. With
    ``seq_split = C > 1`` (``v`` must be 1) every micro-batch is ``C`` sequence chunks: forward units are numbered
    ``m * C + c``, the ``b``-th backward handles unit ``seq_bwd_unit(b, C)``, and the warm-up grows by ``C - 1``
    forwards so that the last chunk of a micro-batch has run forward before its first backward is due."""
    if v > 1 and n % pp != 0:
        raise ValueError(f"interleaved schedule needs micro-batches ({n}) to be a multiple of pipeline stages ({pp})")
    if seq_split > 1 and v > 1:
        raise ValueError("the sequence pipeline does not combine with interleaved model chunks")
    n = n * seq_split
    total = n * v
    warm = min((pp - rank - 1) * (2 if v > 1 else 1) + (v - 1) * pp + (seq_split - 1), total)

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


def _forward_step(model, mb, input_tensor, num_microbatches, collect, loss_scale, carry=None):
    """One micro-batch forward on one model chunk; returns what must be sent on / differentiated. ``carry``: the
    ``KVCarry`` of this micro-batch when ``mb`` is one sequence chunk of it."""
    if input_tensor is not None:
        model.set_input_tensor(input_tensor)
    if carry is not None:
        from .layers.attention import AttnMeta
        B, S = mb["input_ids"].shape
        carry.begin_chunk(int(mb["seq_chunk"]), int(mb["seq_chunk"]) * S)
        meta = AttnMeta(batch=B, seq_len=S, kv_carry=carry)
        out = model(mb["input_ids"], mb.get("labels"), mb.get("loss_mask"), mb.get("position_ids"), attn_meta=meta)
    else:
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


def _backward_step(input_tensor, output, aux, output_grad, carry=None, chunk: int = 0):
    if input_tensor is not None and input_tensor.grad is not None:
        input_tensor.grad = None
    tensors, grads = [output], [output_grad]          # last stage: the output is the scaled loss, its gradient is 1
    if aux is not None and output_grad is not None:
        tensors.append(aux)
        grads.append(torch.ones_like(aux))
    if carry is not None:
        # gradients that the later chunks of this micro-batch left for this chunk's keys and values
        roots, root_grads = carry.roots_and_grads(chunk)
        tensors += roots
        grads += root_grads
    if output_grad is None and len(tensors) == 1:
        output.backward()
    else:
        if grads[0] is None:
            grads[0] = torch.ones_like(output)
        torch.autograd.backward(tensors, grads)
    if carry is not None:
        carry.release(chunk)
    return None if input_tensor is None else input_tensor.grad


def forward_backward_no_pipelining(model, microbatches: List[dict], loss_scale: float = 1.0, seq_split: int = 1):
    """All micro-batches on one stage. With ``seq_split = C > 1`` each micro-batch runs as ``C`` sequence chunks: all
    chunks forward (keys / values carried along), then backward last chunk first; activation memory of everything but
    the keys and values is that of one chunk."""
    losses: List[torch.Tensor] = []
    n = len(microbatches)
    if seq_split <= 1:
        for mb in microbatches:
            out, _ = _forward_step(model, mb, None, n, losses, loss_scale)
            out.backward()
        return losses
    from ..modules.seq_pipe import KVCarry, SequenceSplit
    splitter = SequenceSplit(seq_split)
    for mb in microbatches:
        carry, outs, parts = KVCarry(), [], []
        for part in splitter.split(mb):
            out, _ = _forward_step(model, part, None, n * seq_split, parts, loss_scale, carry)
            outs.append(out)
        for c in reversed(range(seq_split)):
            _backward_step(None, outs[c], None, None, carry, c)
        losses.append(torch.stack(parts).mean())
    return losses


def run_schedule(chunks: List[torch.nn.Module], microbatches: List[dict], hidden_shape, dtype,
                 loss_scale: float = 1.0, seq_split: int = 1) -> List[torch.Tensor]:
    """Execute this rank's schedule (``build_schedule``) over its model chunks; returns the micro-batch losses on
    the rank that holds the last chunk of the last stage. ``seq_split = C > 1``: sequence pipeline — every micro-batch
    enters as ``C`` sequence chunks (``hidden_shape`` is that of one chunk), each stage keeps the keys and values of
    the chunks it has seen, and a micro-batch's chunks run backward in reverse order."""
    pp = ps.get_pipeline_model_parallel_world_size()
    rank = ps.get_pipeline_model_parallel_rank()
    v, n = len(chunks), len(microbatches)
    if seq_split > 1:
        from ..modules.seq_pipe import KVCarry, SequenceSplit
        splitter = SequenceSplit(seq_split)
        units = [part for mb in microbatches for part in splitter.split(mb)]
        carries = [KVCarry() for _ in microbatches]
        return _run_seq_schedule(chunks[0], units, carries, hidden_shape, dtype, loss_scale, seq_split, pp, rank)
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


def _run_seq_schedule(model, units, carries, hidden_shape, dtype, loss_scale, C, pp, rank) -> List[torch.Tensor]:
    """``run_schedule`` for the sequence pipeline (one model chunk per rank). Forward unit ``u`` is chunk ``u % C`` of
    micro-batch ``u // C``; the ``b``-th backward handles unit ``seq_bwd_unit(b, C)``. Returns one loss per micro-batch
    (the mean of its chunk losses) on the last stage."""
    n_units = len(units)
    steps = build_schedule(pp, 1, n_units // C, rank, seq_split=C)
    dev = next(model.parameters()).device
    comm = P2PCommunicator(hidden_shape, dtype, dev)
    parts: List[torch.Tensor] = []
    kept: Dict[int, tuple] = {}             # forward unit -> (input, output, aux)
    act_pending = grad_pending = None
    act_in: Dict[int, torch.Tensor] = {}
    grad_in: Dict[int, torch.Tensor] = {}
    act_owner = grad_owner = None

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

    for st in steps:
        y = gx = None
        if st.fwd is not None:
            if act_owner is not None:
                finish_act(act_owner)
                act_owner = None
            u = st.fwd
            x = act_in.pop(u, None)
            y, aux = _forward_step(model, units[u], x, n_units, parts, loss_scale, carries[u // C])
            kept[u] = (x, y, aux)
        if st.send_act is not None or st.recv_act is not None:
            if act_owner is not None:
                finish_act(act_owner)
            act_pending = comm.exchange_act(y if st.send_act is not None else None, st.recv_act is not None)
            act_owner = st
        if st.bwd is not None:
            if grad_owner is not None:
                finish_grad(grad_owner)
                grad_owner = None
            b = st.bwd
            u = seq_bwd_unit(b, C)
            g = grad_in.pop(b, None)
            xi, yo, au = kept.pop(u)
            gx = _backward_step(xi, yo, au, g, carries[u // C], u % C)
        if st.send_grad is not None or st.recv_grad is not None:
            if grad_owner is not None:
                finish_grad(grad_owner)
            grad_pending = comm.exchange_grad(gx if st.send_grad is not None else None, st.recv_grad is not None)
            grad_owner = st
    if act_owner is not None:
        finish_act(act_owner)
    if grad_owner is not None:
        finish_grad(grad_owner)
    run_schedule.last_bytes_sent = comm.bytes_sent
    if not parts:
        return []
    per_mb = torch.stack(parts).view(-1, C).mean(dim=1)
    return list(per_mb)


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
                 overlap: bool = True, seq_split_num: int = 1):
        self.chunks = list(chunks)
        self.optimizer, self.mbs, self.loss_scale, self.overlap = optimizer, micro_batch_size, loss_scale, overlap
        self.seq_split = int(seq_split_num or 1)
        if self.seq_split > 1 and len(self.chunks) > 1:
            raise ValueError("seq_split_num > 1 (sequence pipeline) does not combine with pp_interleave_num > 1")
        if self.seq_split > 1 and ps.get_context_parallel_world_size() > 1:
            raise ValueError("seq_split_num > 1 (sequence pipeline) does not combine with context parallelism")

    def __call__(self, batch: Dict[str, torch.Tensor]):
        cfg = self.chunks[0].config
        n = batch["input_ids"].shape[0] // self.mbs
        mbs = [{k: v[i * self.mbs:(i + 1) * self.mbs] for k, v in batch.items() if v is not None} for i in range(n)]
        S = batch["input_ids"].shape[1]
        tp = ps.get_tensor_model_parallel_world_size()
        if S % self.seq_split:
            raise ValueError(f"sequence length {S} is not divisible by seq_split_num {self.seq_split}")
        T = self.mbs * (S // self.seq_split) // (tp if cfg.sequence_parallel else 1)
        shape = (T, cfg.hidden_size)
        dtype = cfg.compute_dtype if isinstance(cfg.compute_dtype, torch.dtype) else getattr(torch, str(cfg.compute_dtype))
        self.optimizer.zero_grad()
        if len(self.chunks) > 1:
            losses = forward_backward_pipelining_with_interleaving(self.chunks, mbs, shape, dtype, self.loss_scale, self.overlap)
        elif ps.get_pipeline_model_parallel_world_size() > 1:
            losses = run_schedule([self.chunks[0]], mbs, shape, dtype, self.loss_scale, self.seq_split)
        else:
            losses = forward_backward_no_pipelining(self.chunks[0], mbs, self.loss_scale, self.seq_split)
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
