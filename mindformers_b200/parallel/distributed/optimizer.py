"""Sharded AdamW over flat buffers (ZeRO-1 style distributed optimizer).

Each data-parallel rank owns ``1/dp`` of every flat buffer: its slice of the fp32 gradient arrives by
reduce-scatter, the fused kernel updates the bf16 parameters (+16-bit master remainder) and the fp32
moments of that slice, and an all-gather publishes the new parameters. Global-norm clipping and the
skip-on-spike / skip-on-NaN decision are read from a device scalar, so a step has no host
synchronisation. Semantics follow the reference: ``core/optim/adamw.py:38-66`` (decoupled decay, bias
correction, eps outside the square root), ``core/clip_grad.py:60-101`` (coefficient ``max_norm/(norm+1e-6)``
applied only when the norm exceeds ``max_norm``), skip-data in ``wrapper/wrapper.py:276-281``.
State names for checkpoints are ``adam_m.<param>`` / ``adam_v.<param>`` and ``global_step``.
"""
from __future__ import annotations

import math
import os
import re
from typing import Callable, Dict, Optional, Union

import torch
import torch.distributed as dist

from ...ops import _lib
from ...ops import functional as Fn
from .. import fused_comm, symm_mem
from .. import parallel_state as ps
from .param_grad_buffer import ParamAndGradBuffer, build_buffers


class _Shard:
    def __init__(self, buf: ParamAndGradBuffer, group, world: int, rank: int):
        self.buf, self.group, self.world, self.rank = buf, group, world, rank
        n = buf.ranges.numel
        if n % world != 0:
            raise ValueError(f"buffer {buf.name} ({n} elements) is not divisible by the shard count {world}")
        self.len = n // world
        self.begin = rank * self.len
        self.end = self.begin + self.len
        dev = buf.param_data.device
        self.param = buf.param_data[self.begin:self.end]
        self.grad = buf.grad_data[self.begin:self.end]
        self.m = torch.zeros(self.len, dtype=torch.float32, device=dev)
        self.v = torch.zeros(self.len, dtype=torch.float32, device=dev)
        self.bf16 = buf.param_data.dtype == torch.bfloat16
        if self.bf16:
            self.lo = torch.zeros(self.len, dtype=torch.int16, device=dev)
        else:
            self.lo = None
            self.master = self.param.float().clone() if buf.param_data.dtype != torch.float32 else None

    def clip(self, lo, hi):
        return max(0, min(hi, self.end) - max(lo, self.begin))

    def local(self, lo, hi):
        a, b = max(lo, self.begin), min(hi, self.end)
        if b <= a:
            return None
        return a - self.begin, b - self.begin


class DistributedOptimizer:
    """AdamW over the flat buffers of ``model``.

    Args:
        learning_rate: float or a callable ``step -> lr`` (steps count from 1).
        max_grad_norm: clip threshold (0 disables); skip_threshold: skip the update when the global norm
        is at least this (0 disables); non-finite norms always skip.
    """

    def __init__(self, model: torch.nn.Module, *, learning_rate: Union[float, Callable[[int], float]] = 1e-4,
                 betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0, max_grad_norm: float = 1.0,
                 skip_threshold: float = 0.0, grad_dtype: torch.dtype = torch.float32,
                 tensor_parallel: Optional[int] = None, sequence_parallel: bool = False,
                 shard_optimizer: bool = True, fused_dp_comm: Optional[bool] = None):
        self.model = model
        self.lr = learning_rate
        self.beta1, self.beta2 = betas
        self.eps, self.wd = eps, weight_decay
        self.max_grad_norm, self.skip_threshold = max_grad_norm, skip_threshold
        self.global_step = 0
        self.tp = tensor_parallel if tensor_parallel is not None else ps.get_tensor_model_parallel_world_size()
        self.sequence_parallel = sequence_parallel
        dp = ps.get_data_parallel_world_size(with_context_parallel=True) if shard_optimizer else 1
        edp = ps.get_expert_data_parallel_world_size() if shard_optimizer else 1
        first = next(p for p in model.parameters() if p.requires_grad)
        if fused_dp_comm is None:
            fused_dp_comm = fused_comm.dp_enabled() and max(dp, edp) > 1
        self.fused_dp = bool(fused_dp_comm) and first.is_cuda and first.dtype == torch.bfloat16 \
            and grad_dtype == torch.float32 and max(dp, edp) <= 8
        self._symm: Dict[str, object] = {}

        def symm_alloc(tag, numel, dt, dev):
            grp = ps.get_expert_data_parallel_group() if tag.startswith("expert") else \
                ps.get_data_parallel_group(with_context_parallel=True)
            world = edp if tag.startswith("expert") else dp
            if world <= 1:
                return torch.zeros(numel, dtype=dt, device=dev)
            buf = symm_mem.allocate(f"dpopt.{tag}.{id(self)}", numel * torch.empty((), dtype=dt).element_size(), grp, dev)
            t = buf.tensor.view(dt)[:numel]
            t.zero_()
            self._symm[tag] = buf
            return t

        self.buffers = build_buffers(model, tp=self.tp, sequence_parallel=sequence_parallel, grad_dtype=grad_dtype,
                                     dense_pad=dp, expert_pad=edp, allocator=symm_alloc if self.fused_dp else None)
        self.shards: Dict[str, _Shard] = {}
        for name, buf in self.buffers.items():
            if name.startswith("expert"):
                grp, world, rank = ps.get_expert_data_parallel_group(), edp, ps.get_expert_data_parallel_rank() if edp > 1 else 0
            else:
                grp, world = ps.get_data_parallel_group(with_context_parallel=True), dp
                rank = ps.get_data_parallel_rank(with_context_parallel=True) if dp > 1 else 0
            self.shards[name] = _Shard(buf, grp, world, rank)
        dev = next(iter(self.buffers.values())).param_data.device
        self.sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self._dup_sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self.skipped = torch.zeros(1, dtype=torch.int32, device=dev)
        # the fp32 master starts as the exact value of the bf16 parameter, i.e. remainder 0
        self._dp_epoch = 0
        self._overlap = None          # state of the bucketed reduction that runs under the backward pass
        self.overlap_grad_reduce = os.environ.get("MFB_DP_OVERLAP", "1") != "0"
        # opt-in: AdamW + publication of the new parameters run on the side stream in the order the next forward pass
        # needs them, and that forward pass waits per group of layers instead of at the end of the step
        self.overlap_param_gather = os.environ.get("MFB_DP_PARAM_OVERLAP", "0") == "1"
        self._pub = None              # pending publication: events per row, rows already waited for
        if self.fused_dp:
            self._setup_fused_dp(dev)
            self._setup_overlap(dev)

    def _setup_fused_dp(self, dev):
        """Peer pointer tables and flag words of the fused reduce-scatter / AdamW / all-gather kernels."""
        import ctypes
        lib = _lib.get_lib()
        words = lib.mfb_dp_flag_words()
        self._dp_scratch = torch.zeros(lib.mfb_dp_reduce_scratch(), dtype=torch.float32, device=dev)
        for name, sh in self.shards.items():
            sh.fused = False
            if sh.world <= 1 or not sh.bf16 or f"{name}.grad" not in self._symm:
                continue      # fp32 parameter buffers (router weights) keep the NCCL reduce-scatter / all-gather
            flags = symm_mem.allocate(f"dpopt.{name}.flags.{id(self)}", words * 4, sh.group, dev)
            flags.tensor.zero_()
            arr = ctypes.c_longlong * sh.world
            sh.peer_grad = arr(*[int(p) for p in self._symm[f"{name}.grad"].ptrs])
            sh.peer_param = arr(*[int(p) for p in self._symm[f"{name}.param"].ptrs])
            sh.peer_flags = arr(*[int(p) for p in flags.ptrs])
            sh.flags = flags
            sh.fused = True
        torch.cuda.synchronize()
        if dist.is_initialized():
            dist.barrier()      # every rank's flag words are zero before anyone's first step

    # ---------------------------------------------------------------------------------------------
    # Gradient reduction under the backward pass (the reference overlaps the data-parallel gradient reduction with
    # the backward pass through MindSpore's ``enable_parallel_optimizer`` + ``parallel_speed_up.json``
    # ``enable_grad_comm_opt``; wrapper/wrapper.py:255,560).
    def _setup_overlap(self, dev):
        """Finds, per fused buffer, the flat-buffer range of every decoder layer. The weight matrices of a layer are
        consecutive in the buffer (same category, registration order), so a layer's range is final as soon as the
        backward pass has left the layer. Everything else (embedding, head, norms, biases) stays with the pass
        that follows the backward pass."""
        from ..layers.transformer_layer import TransformerBlock
        blocks = [(n, m) for n, m in self.model.named_modules() if isinstance(m, TransformerBlock) and len(m.layers)]
        self._ov_blocks, self._ov_layers = [], {}
        self._ov_stream = torch.cuda.Stream(device=dev)
        self._pub_skipped = torch.zeros(1, dtype=torch.int32, device=dev)
        # whoever reads the parameters next (a forward pass, a checkpoint) first waits for a publication in flight
        self.model._mfb_param_sync = self.finish_param_gather
        self.model.register_forward_pre_hook(lambda _m, _a: self._before_model_forward())
        if len(blocks) != 1:
            return
        prefix, block = blocks[0]
        pat = re.compile(r"^" + re.escape(prefix + "." if prefix else "") + r"layers\.(\d+)\.")
        rows = _lib.get_lib().mfb_dp_bucket_rows()
        for name, sh in self.shards.items():
            if not getattr(sh, "fused", False):
                continue
            span: Dict[int, list] = {}
            main_end = min(sh.buf.ranges.dup_begin, sh.buf.ranges.decay_end) if self.tp > 1 else sh.buf.ranges.decay_end
            for pname, _, off, cnt in sh.buf.entries:
                mt = pat.match(pname)
                if mt is None or off >= main_end:
                    continue
                gid = int(mt.group(1))
                end = (off + cnt + 127) // 128 * 128
                lo_hi = span.setdefault(gid, [off, end])
                lo_hi[0], lo_hi[1] = min(lo_hi[0], off), max(lo_hi[1], end)
            ids = sorted(span)
            # the ranges must tile one interval in layer order, otherwise a "final" range could hold other gradients
            ok = bool(ids) and all(span[a][1] == span[b][0] for a, b in zip(ids, ids[1:]))
            inside = sum(cnt for pname, _, off, cnt in sh.buf.entries
                         if ids and span[ids[0]][0] <= off < span[ids[-1]][1] and pat.match(pname) is None)
            if not ok or inside:
                continue
            group = max(1, -(-len(ids) // rows))              # layers per bucket, so that the rows suffice
            self._ov_layers[name] = {"span": span, "ids": ids, "group": group}
        if self._ov_layers:
            self._ov_blocks = [block]
            self._ov_scratch = torch.zeros(_lib.get_lib().mfb_dp_reduce_scratch(), dtype=torch.float32, device=dev)
            self._ov_sumsq = torch.zeros(1, dtype=torch.float32, device=dev)

    def _before_model_forward(self):
        """A forward pass that starts while parameters are still being published: the parameters outside the decoder
        layers are needed at once, the layers wait one by one (a forward pass outside the training step included)."""
        if self._pub is None:
            return
        self._wait_published(0)
        self._wait_published(1)
        if self._pub is not None:
            for b in getattr(self, "_ov_blocks", []):
                b.params_ready_hook = self._layer_params_needed

    def begin_grad_overlap(self):
        """Call before the forward pass of the step's last micro-batch: from then on each decoder layer's gradient
        range is reduced over the data-parallel group as soon as the backward pass has finished the layer."""
        self._overlap = None
        if not (self.fused_dp and self.overlap_grad_reduce and getattr(self, "_ov_layers", None)):
            return
        if not all(getattr(self.shards[n], "fused", False) for n in self._ov_layers):
            return                            # the shards are on the NCCL path (set_fused_dp(False))
        self._dp_epoch += 1
        self._ov_sumsq.zero_()
        self._overlap = {"row": 0, "low": {n: None for n in self._ov_layers}, "pending": {n: [] for n in self._ov_layers},
                         "event": None}
        for b in self._ov_blocks:
            b.grads_final_hook = self._layer_grads_final

    def _layer_grads_final(self, gid: int):
        ov = self._overlap
        if ov is None or ov.get("stopped"):
            return
        lib = _lib.get_lib()
        for name, info in self._ov_layers.items():
            if gid not in info["span"]:
                continue
            pend = ov["pending"][name]
            pend.append(gid)
            first = gid == info["ids"][0]
            if len(pend) < info["group"] and not first:
                continue
            lo = min(info["span"][g][0] for g in pend)
            hi = max(info["span"][g][1] for g in pend)
            pend.clear()
            if ov["low"][name] is not None and hi != ov["low"][name]:
                ov["stopped"] = True          # layers finished out of order: leave the rest to the closing pass
                return
            sh = self.shards[name]
            row = ov["row"]
            ov["row"] += 1
            rc = lib.mfb_dp_announce(sh.world, sh.rank, self._dp_epoch, row, sh.peer_flags, _lib.stream_ptr())
            _lib.check(rc, "mfb_dp_announce")
            ev = torch.cuda.Event()
            ev.record()
            a, b = max(lo, sh.begin), min(hi, sh.end)
            n = max(0, b - a)
            self._ov_stream.wait_event(ev)
            with torch.cuda.stream(self._ov_stream):
                rc = lib.mfb_dp_reduce_bucket(sh.world, sh.rank, self._dp_epoch, row, a if n else 0, n, sh.peer_grad,
                                              sh.peer_flags, sh.buf.grad_data.data_ptr() + 4 * (a if n else 0),
                                              self._ov_scratch.data_ptr(), self._ov_sumsq.data_ptr(), 148,
                                              _lib.status_word(sh.grad.device).data_ptr(), _lib.stream_ptr())
            _lib.check(rc, "mfb_dp_reduce_bucket")
            _lib.count_launch(4 if n else 2)
            ov["low"][name] = lo
            ov.setdefault("high", {}).setdefault(name, hi)

    def _end_grad_overlap(self):
        """Joins the side stream and returns, per buffer, the range that the buckets have covered."""
        ov, self._overlap = self._overlap, None
        for b in getattr(self, "_ov_blocks", []):
            b.grads_final_hook = None
        if ov is None:
            return {}
        torch.cuda.current_stream().wait_stream(self._ov_stream)
        return {n: (lo, ov["high"][n]) for n, lo in ov["low"].items() if lo is not None}

    def zero_grad(self, set_to_none: bool = True):
        pub = self._pub
        if pub is not None:
            # the embedding, head and norm parameters are needed first, and their publication by every rank also says
            # that every rank has finished reading this rank's gradients: only now may they be overwritten
            self._wait_published(0)
            self._wait_published(1)
            for name, buf in self.buffers.items():
                sh = self.shards[name]
                if name in pub["shards"]:
                    buf.grad_data[:sh.begin].zero_()      # this rank's own slice is zeroed by its AdamW pieces
                    buf.grad_data[sh.end:].zero_()
                else:
                    buf.zero_grad()
            for b in getattr(self, "_ov_blocks", []):
                b.params_ready_hook = self._layer_params_needed
        else:
            for buf in self.buffers.values():
                buf.zero_grad()
        for p in self.model.parameters():
            p.grad = None

    # ---- parameter publication under the next forward pass ----------------------------------------------------------
    def _publish_rows(self, name):
        """``[(row, lo, hi)]`` in the order the forward pass needs the parameters: rows 0 / 1 = everything outside the
        decoder layers (below / above their range), rows 2.. = groups of layers in ascending order."""
        sh = self.shards[name]
        info = getattr(self, "_ov_layers", {}).get(name)
        if info is None:
            return [(0, sh.begin, sh.end), (1, sh.end, sh.end)]
        ids, span = info["ids"], info["span"]
        d0, d1 = span[ids[0]][0], span[ids[-1]][1]
        rows = [(0, 0, d0), (1, d1, sh.buf.ranges.numel)]
        per = max(1, -(-len(ids) // 60))
        for gi, i in enumerate(range(0, len(ids), per)):
            grp = ids[i:i + per]
            rows.append((2 + gi, span[grp[0]][0], span[grp[-1]][1]))
        return rows

    def _row_of_layer(self, name, gid):
        info = self._ov_layers[name]
        per = max(1, -(-len(info["ids"]) // 60))
        return 2 + info["ids"].index(gid) // per

    def _wait_published(self, row: int):
        pub = self._pub
        if pub is None or row in pub["waited"]:
            return
        pub["waited"].add(row)
        lib = _lib.get_lib()
        for name in pub["shards"]:
            ev = pub["events"][name].get(row)
            if ev is None:
                continue
            torch.cuda.current_stream().wait_event(ev)        # this GPU's own pieces: ordered by the event
            sh = self.shards[name]
            rc = lib.mfb_dp_wait_published(sh.world, sh.rank, pub["epoch"], row, sh.peer_flags,
                                           _lib.status_word(sh.grad.device).data_ptr(), _lib.stream_ptr())
            _lib.check(rc, "mfb_dp_wait_published")
            _lib.count_launch(1)
        if len(pub["waited"]) >= pub["rows"]:
            self._pub = None
            for b in getattr(self, "_ov_blocks", []):
                b.params_ready_hook = None

    def _layer_params_needed(self, gid: int):
        pub = self._pub
        if pub is None:
            return
        for name in pub["shards"]:
            if name in self._ov_layers and gid in self._ov_layers[name]["span"]:
                self._wait_published(self._row_of_layer(name, gid))

    def finish_param_gather(self):
        """Make the current stream wait for every parameter that is still being published (call before anything other
        than the next training step reads the parameters: evaluation, generation, a checkpoint)."""
        pub = self._pub
        if pub is None:
            return
        for row in range(pub["rows"]):
            self._wait_published(row)
        self._pub = None
        for b in getattr(self, "_ov_blocks", []):
            b.params_ready_hook = None

    def _step_published(self, lr, grad_scale):
        """AdamW and publication of the fused shards piece by piece on the side stream (see ``overlap_param_gather``)."""
        lib = _lib.get_lib()
        main = torch.cuda.current_stream()
        # the skip decision of the step, on the compute stream (the pieces reach the same verdict from the same scalar)
        nrm = self.sumsq.sqrt() * abs(grad_scale)
        bad = ~torch.isfinite(self.sumsq)
        if self.skip_threshold > 0:
            bad = bad | (nrm >= self.skip_threshold)
        self.skipped.copy_(bad.to(torch.int32))
        ready = torch.cuda.Event()
        ready.record(main)
        self._ov_stream.wait_event(ready)
        pub = {"epoch": self._dp_epoch, "events": {}, "waited": set(), "shards": [], "rows": 0}
        bc1, bc2 = 1.0 - self.beta1 ** self.global_step, 1.0 - self.beta2 ** self.global_step
        scratch_skipped = self._pub_skipped
        with torch.cuda.stream(self._ov_stream):
            for name, sh in self.shards.items():
                if not getattr(sh, "fused", False):
                    continue
                pub["shards"].append(name)
                pub["events"][name] = {}
                r = sh.buf.ranges
                d_end = max(0, min(r.decay_end, sh.end) - sh.begin)
                rows = self._publish_rows(name)
                pub["rows"] = max(pub["rows"], len(rows))
                for row, lo, hi in rows:
                    a, b = max(lo, sh.begin), min(hi, sh.end)
                    n = max(0, b - a)
                    off = a - sh.begin if n else 0
                    rc = lib.mfb_dp_adamw_publish(
                        sh.world, sh.rank, self._dp_epoch, row, a if n else sh.begin, n, off, sh.peer_param, sh.peer_flags,
                        sh.lo.data_ptr(), sh.m.data_ptr(), sh.v.data_ptr(), sh.grad.data_ptr(), self.sumsq.data_ptr(),
                        scratch_skipped.data_ptr(), d_end, lr, self.beta1, self.beta2, self.eps, self.wd, bc1, bc2,
                        self.max_grad_norm, self.skip_threshold, grad_scale, _lib.status_word(sh.grad.device).data_ptr(),
                        _lib.stream_ptr())
                    _lib.check(rc, "mfb_dp_adamw_publish")
                    _lib.count_launch(1)
                    ev = torch.cuda.Event()
                    ev.record()
                    pub["events"][name][row] = ev
        self._pub = pub

    def current_lr(self) -> float:
        return float(self.lr(self.global_step) if callable(self.lr) else self.lr)

    # ---------------------------------------------------------------------------------------------
    def reduce_gradients(self):
        """Fold stray autograd grads, all-reduce SP-replicated grads over TP, reduce-scatter over DP."""
        tp_group = ps.get_tensor_model_parallel_group()
        for name, buf in self.buffers.items():
            buf.collect_autograd_grads()
            r = buf.ranges
            if self.tp > 1 and self.sequence_parallel and r.sp_end > r.sp_begin and tp_group is not None:
                dist.all_reduce(buf.grad_data[r.sp_begin:r.sp_end], group=tp_group)
            sh = self.shards[name]
            if sh.world > 1 and not getattr(sh, "fused", False):
                dist.reduce_scatter_tensor(sh.grad, buf.grad_data, op=dist.ReduceOp.SUM, group=sh.group)

    def _global_sumsq(self, covered=None):
        self.sumsq.zero_()
        self._dup_sumsq.zero_()
        if covered:
            self.sumsq.add_(self._ov_sumsq)      # squared norm of the ranges that were reduced under the backward pass
        for name, sh in self.shards.items():
            if getattr(sh, "fused", False):
                # reduce-scatter by peer loads; the squared norm of the reduced slice comes out of the same pass
                lo, hi = (covered or {}).get(name, (sh.end, sh.end))
                pieces = [(sh.begin, min(sh.end, lo)), (max(sh.begin, hi), sh.end)] if lo < hi else [(sh.begin, sh.end)]
                pieces = [(a, b) for a, b in pieces if b > a] or [(sh.begin, sh.begin)]    # the announce must still go out
                for a, b in pieces:
                    rc = _lib.get_lib().mfb_dp_reduce(sh.world, sh.rank, self._dp_epoch, a, b - a, sh.peer_grad,
                                                      sh.peer_flags, sh.buf.grad_data.data_ptr() + 4 * a,
                                                      self._dp_scratch.data_ptr(), self.sumsq.data_ptr(), 1,
                                                      _lib.status_word(sh.grad.device).data_ptr(), _lib.stream_ptr())
                    _lib.check(rc, "mfb_dp_reduce")
                    _lib.count_launch(2)
            else:
                Fn.grad_sumsq(sh.grad, self.sumsq, accumulate=True)
            r = sh.buf.ranges
            loc = sh.local(r.dup_begin, r.dup_end) if self.tp > 1 else None
            if loc is not None:
                Fn.grad_sumsq(sh.grad[loc[0]:loc[1]], self._dup_sumsq, accumulate=True)
        if self.tp > 1:
            # TP-replicated parameters appear on every TP rank: count them once
            self.sumsq.sub_(self._dup_sumsq * (1.0 - 1.0 / self.tp))
        world = ps.get_world_group()
        if world is not None and dist.is_initialized() and dist.get_world_size() > 1:
            # every rank's shard is disjoint across DP; TP/PP ranks hold different parameters
            dist.all_reduce(self.sumsq, group=world)
        return self.sumsq

    def set_fused_dp(self, flag: bool):
        """Switch the shards that were set up for the peer-memory reduce-scatter / AdamW / all-gather kernels
        between those kernels and the NCCL collectives (the buffers serve both). Every rank must switch at the
        same step. Used by the benchmark to time the library path on the same engine."""
        for sh in self.shards.values():
            if not hasattr(sh, "_fused_capable"):
                sh._fused_capable = bool(getattr(sh, "fused", False))
            sh.fused = bool(flag) and sh._fused_capable

    def reduce_and_norm(self) -> torch.Tensor:
        """Gradient reduction (tensor-parallel replicas, data-parallel reduce-scatter) and the squared global
        norm of the reduced gradients, without the parameter update: the first half of ``step``."""
        started = self._overlap is not None      # begin_grad_overlap has already opened this step's epoch
        covered = self._end_grad_overlap()
        if not started:
            self._dp_epoch += 1
        self.reduce_gradients()
        return self._global_sumsq(covered)

    def step(self, grad_scale: float = 1.0):
        """One optimizer step. ``grad_scale`` multiplies the gradients (1/dp averaging, loss-scale inverse)."""
        self.finish_param_gather()          # a step whose forward pass never ran (tests) still owes the waits
        self.reduce_and_norm()
        self.global_step += 1
        lr = self.current_lr()
        self.skipped.zero_()
        deferred = self.overlap_param_gather and self.fused_dp and hasattr(self, "_ov_stream") \
            and any(getattr(sh, "fused", False) for sh in self.shards.values())
        if deferred:
            self._step_published(lr, grad_scale)
        for name, sh in self.shards.items():
            r = sh.buf.ranges
            d_end = max(0, min(r.decay_end, sh.end) - sh.begin)
            if getattr(sh, "fused", False) and deferred:
                continue
            if getattr(sh, "fused", False):
                bc1, bc2 = 1.0 - self.beta1 ** self.global_step, 1.0 - self.beta2 ** self.global_step
                rc = _lib.get_lib().mfb_dp_adamw_allgather(
                    sh.world, sh.rank, self._dp_epoch, sh.begin, sh.len, sh.peer_param, sh.peer_flags, sh.lo.data_ptr(),
                    sh.m.data_ptr(), sh.v.data_ptr(), sh.grad.data_ptr(), self.sumsq.data_ptr(), self.skipped.data_ptr(),
                    d_end, lr, self.beta1, self.beta2, self.eps, self.wd, bc1, bc2, self.max_grad_norm,
                    self.skip_threshold, grad_scale, _lib.status_word(sh.grad.device).data_ptr(), _lib.stream_ptr())
                _lib.check(rc, "mfb_dp_adamw_allgather")
                _lib.count_launch(2)
                continue
            if sh.bf16:
                Fn.adamw_step(sh.param, sh.lo, sh.m, sh.v, sh.grad, lr=lr, beta1=self.beta1, beta2=self.beta2,
                              eps=self.eps, weight_decay=self.wd, step=self.global_step, decay_end=d_end,
                              sumsq=self.sumsq, skipped=self.skipped, max_norm=self.max_grad_norm,
                              skip_threshold=self.skip_threshold, grad_scale=grad_scale)
            else:
                self._step_fp32(sh, lr, d_end, grad_scale)
            if sh.world > 1:
                dist.all_gather_into_tensor(sh.buf.param_data, sh.param.clone(), group=sh.group)
        return self.sumsq

    def _step_fp32(self, sh: _Shard, lr, d_end, grad_scale):
        ss = self.sumsq
        nrm = ss.sqrt() * abs(grad_scale)
        bad = ~torch.isfinite(ss)
        if self.skip_threshold > 0:
            bad = bad | (nrm >= self.skip_threshold)
        clip = torch.ones_like(nrm)
        if self.max_grad_norm > 0:
            clip = torch.where(nrm >= self.max_grad_norm, self.max_grad_norm / (nrm + 1e-6), clip)
        keep = (~bad).float()
        g = sh.grad.float() * (clip * grad_scale)
        t = self.global_step
        bc1, bc2 = 1 - self.beta1 ** t, 1 - self.beta2 ** t
        m_new = self.beta1 * sh.m + (1 - self.beta1) * g
        v_new = self.beta2 * sh.v + (1 - self.beta2) * g * g
        w = sh.master if sh.master is not None else sh.param
        w_new = w.clone()
        w_new[:d_end] *= (1 - lr * self.wd)
        w_new -= (lr / bc1) * m_new / ((v_new / bc2).sqrt() + self.eps)
        sh.m.copy_(torch.where(bad, sh.m, m_new))
        sh.v.copy_(torch.where(bad, sh.v, v_new))
        w.copy_(torch.where(bad, w, w_new))
        if sh.master is not None:
            sh.param.copy_(w)
        self.skipped.add_(bad.to(torch.int32))
        del keep

    # ---------------------------------------------------------------------------------------------
    def global_norm(self, grad_scale: float = 1.0) -> torch.Tensor:
        """Norm of the last step's gradients (device scalar)."""
        return self.sumsq.sqrt() * abs(grad_scale)

    def state_norms(self) -> Dict[str, float]:
        """L2 norms of this rank's moment shards (for ``TrainingStateMonitor``)."""
        out = {}
        for name, sh in self.shards.items():
            out[f"{name}.adam_m"] = float(sh.m.norm())
            out[f"{name}.adam_v"] = float(sh.v.norm())
        return out

    # ---- checkpoint -------------------------------------------------------------------------------
    def state_dict(self) -> dict:
        """Per-parameter optimizer state of this rank's shard, keyed like the reference's checkpoints.
        Values are flat slices ``(tensor, offset_in_param)`` so that shards can be merged on load."""
        out = {"global_step": self.global_step, "shards": {}}
        for name, sh in self.shards.items():
            out["shards"][name] = {"begin": sh.begin, "end": sh.end, "m": sh.m, "v": sh.v,
                                   "lo": sh.lo, "master": getattr(sh, "master", None)}
        return out

    def named_states(self) -> Dict[str, torch.Tensor]:
        """``adam_m.<param>`` / ``adam_v.<param>`` (and ``master_lo.<param>``) of this rank's share of every parameter.
        A rank that owns a whole parameter gives views of the parameter's (tensor-parallel local) shape. Under a
        sharded optimizer a rank owns a flat slice of each buffer, so a parameter that straddles a shard boundary
        comes as a 1-D slice plus ``__slice__.<param>`` = ``[offset, count, numel]`` (int64): where the slice sits
        in the flattened local parameter. Parameters outside the rank's slice are left out; the data-parallel
        peers hold them."""
        out: Dict[str, torch.Tensor] = {}
        for name, sh in self.shards.items():
            for pname, (o, cnt, shape) in sh.buf.index.items():
                lo_, hi_ = max(o, sh.begin), min(o + cnt, sh.end)
                if hi_ <= lo_:
                    continue
                whole = (lo_ == o and hi_ == o + cnt)
                a, b = lo_ - sh.begin, hi_ - sh.begin
                for key, src in (("adam_m", sh.m), ("adam_v", sh.v), ("master_lo", sh.lo)):
                    if src is None:
                        continue
                    out[f"{key}.{pname}"] = src[a:b].view(shape) if whole else src[a:b]
                if not whole:
                    out[f"__slice__.{pname}"] = torch.tensor([lo_ - o, hi_ - lo_, cnt], dtype=torch.int64)
        return out

    def load_named_states(self, states: Dict[str, torch.Tensor], global_step: Optional[int] = None,
                          strict: bool = False, model_params: Optional[Dict[str, torch.Tensor]] = None):
        """Restore the moments (and master remainders) of this rank's slice of every buffer from ``states``.

        A state may be (a) of the parameter's local shape, (b) a 1-D slice with its ``__slice__.<param>`` entry, as
        ``named_states`` of a sharded run writes it, or (c) the full tensor of a merged checkpoint, which is cut for
        this rank's tensor- / expert-parallel position first (``model_params`` maps names to the parameters that
        describe that layout). A slice that does not cover what this rank needs (the checkpoint was written under
        another data-parallel layout and not merged) raises instead of leaving moments at zero."""
        from ...checkpoint.sharding import shard_for_param
        missing = []
        for name, sh in self.shards.items():
            for pname, (o, cnt, shape) in sh.buf.index.items():
                lo_, hi_ = max(o, sh.begin), min(o + cnt, sh.end)
                if hi_ <= lo_:
                    continue
                need_a, need_b = lo_ - o, hi_ - o            # range of the flattened local parameter this rank holds
                for key, dst in (("adam_m", sh.m), ("adam_v", sh.v), ("master_lo", sh.lo)):
                    src = states.get(f"{key}.{pname}")
                    if dst is None:
                        continue
                    if src is None:
                        if key != "master_lo":
                            missing.append(f"{key}.{pname}")
                        continue
                    sl = states.get(f"__slice__.{pname}")
                    if sl is not None and src.dim() == 1 and src.numel() == int(sl[1]):
                        off, n = int(sl[0]), int(sl[1])
                    else:
                        if tuple(src.shape) != tuple(shape):
                            p = (model_params or {}).get(pname)
                            if p is None:
                                raise ValueError(f"optimizer state {key}.{pname} has shape {tuple(src.shape)}, the local "
                                                 f"parameter {tuple(shape)}: pass the model parameters to re-slice it")
                            src = shard_for_param(src, p)
                        off, n = 0, cnt
                        src = src.reshape(-1)
                    if off > need_a or off + n < need_b:
                        raise ValueError(
                            f"optimizer state {key}.{pname} covers elements [{off}, {off + n}) of the parameter, this rank "
                            f"needs [{need_a}, {need_b}): the checkpoint was written under another data-parallel layout; "
                            "merge it first (checkpoint.transform.unify_checkpoints, or auto_trans_ckpt with its strategy files)")
                    dst[lo_ - sh.begin:hi_ - sh.begin].copy_(src[need_a - off:need_b - off].to(dst.device))
        if missing and strict:
            raise KeyError(f"checkpoint lacks optimizer states: {missing[:6]}{' ...' if len(missing) > 6 else ''}")
        if global_step is not None:
            self.global_step = int(global_step)

    def reload_model_params(self):
        """Re-derive the master remainder after parameters were overwritten (checkpoint load)."""
        for sh in self.shards.values():
            if sh.bf16:
                sh.lo.zero_()
            elif sh.master is not None:
                sh.master.copy_(sh.param.float())
