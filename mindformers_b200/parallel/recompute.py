"""Activation recomputation and activation offload for the transformer layers.

Three mechanisms, selected by the ``recompute_config`` / ``swap_config`` sections of a configuration (reference
``parallel_core/training_graph/transformer/utils.py:93-317``, ``tools/register/template.py:317-337``):

* **full recompute** (``recompute: true`` or a per-stage layer count): a layer keeps only its input; its forward is run
  again in backward.
* **selective recompute** (``select_recompute: true`` or a list of regular expressions over the sub-module paths of a
  layer): the layer is checkpointed as well, but while its forward runs the outputs of the *expensive* operations
  (matrix products, attention, expert exchange) are kept in a side cache, and the second run takes them from there
  instead of launching the kernels again. What is really recomputed is everything else: norms, rotary embedding, the
  gated activation, residual adds — the operations the reference lists as its default patterns (``mlp.mul``,
  ``mlp.activation_func.silu``, ``.*.norm``). A pattern that matches a module with an expensive operation (for
  example ``mlp\\.linear_fc1``) removes that module from the cache, so its product is recomputed too. With the shapes
  of Llama-3.1-8B this keeps 68 % of a layer's activation bytes and costs a few elementwise kernels per layer.
* **offload** (``swap: true``, ``layer_swap``): the tensors a layer saves for backward are copied to pinned host memory
  on a side stream and brought back when backward reaches the layer; the copies of layer ``i - 1`` are started when
  backward enters layer ``i`` (``default_prefetch`` layers ahead).

``recompute_slice_activation`` and the communication-recompute switches have no effect here: activations are not
sliced over tensor-parallel ranks beyond what sequence parallelism already does, and the fused GEMM + collective
kernels leave no separate communication output to drop; a warning names the keys that were set.
"""
from __future__ import annotations

import re
import threading
from typing import Callable, Dict, List, Optional, Sequence

import torch
from torch.utils.checkpoint import checkpoint

_tls = threading.local()


class _OutputCache:
    """Outputs of the expensive operations of one checkpointed region, in execution order."""

    def __init__(self):
        self.items: List[object] = []
        self.replaying = False
        self.cursor = 0
        self.bypass = 0          # > 0 inside a module whose operations are to be recomputed, not cached

    def push(self, value):
        self.items.append(value)

    def pop(self):
        value = self.items[self.cursor]
        self.items[self.cursor] = None      # the backward graph now owns the tensors
        self.cursor += 1
        return value


def current_cache() -> Optional[_OutputCache]:
    return getattr(_tls, "cache", None)


STATS = {"computed": 0, "replayed": 0}     # expensive operations run / taken from the cache inside selective regions


def cached_output(compute: Callable[[], object]):
    """Called from the forward of an autograd function that wraps an expensive kernel: computes normally outside a
    selective-recompute region; inside one the result is recorded on the first run and returned from the cache on the
    second (the recomputation), so that only the cheap operations of the region run twice."""
    c = current_cache()
    if c is None or c.bypass:
        return compute()
    if c.replaying:
        STATS["replayed"] += 1
        return c.pop()
    value = compute()
    STATS["computed"] += 1
    c.push(value)
    return value


class _Bypass:
    def __init__(self):
        self.prev = None

    def __enter__(self):
        c = current_cache()
        if c is not None:
            c.bypass += 1
        return self

    def __exit__(self, *exc):
        c = current_cache()
        if c is not None:
            c.bypass -= 1
        return False


def selective_checkpoint(fn: Callable, *args):
    """``fn(*args)`` under activation checkpointing with the outputs of its expensive operations cached."""
    cache = _OutputCache()

    def run(*a):
        prev = getattr(_tls, "cache", None)
        _tls.cache = cache
        try:
            return fn(*a)
        finally:
            _tls.cache = prev
            if not cache.replaying:
                cache.replaying = True     # the next run of `run` is the recomputation in backward

    return checkpoint(run, *args, use_reentrant=False)


def full_checkpoint(fn: Callable, *args):
    return checkpoint(fn, *args, use_reentrant=False)


def mark_recompute_modules(layer: torch.nn.Module, patterns: Sequence[str]) -> List[str]:
    """Sub-modules of ``layer`` whose dotted path fully matches one of ``patterns`` run with the cache bypassed: their
    expensive operations are recomputed like everything else. Returns the matched paths."""
    if not patterns:
        return []
    compiled = [re.compile(p) for p in patterns]
    matched = []
    for name, mod in layer.named_modules():
        if not name or getattr(mod, "_recompute_bypass", False):
            continue
        if any(c.fullmatch(name) for c in compiled):
            mod._recompute_bypass = True
            state = {}

            def pre(m, a, _s=state):
                _s["ctx"] = _Bypass().__enter__()

            def post(m, a, out, _s=state):
                _s.pop("ctx").__exit__(None, None, None)

            mod.register_forward_pre_hook(pre)
            mod.register_forward_hook(post)
            matched.append(name)
    return matched


# --------------------------------------------------------------------------------------------------------------
# offload of saved activations to pinned host memory
# --------------------------------------------------------------------------------------------------------------
class _Handle:
    __slots__ = ("host", "event", "device", "gpu", "layer", "shape", "dtype")


class ActivationOffloader:
    """Saved-tensor hooks that move the activations of selected layers to pinned host memory.

    ``with offloader.layer(i): y = layer(x)`` registers every tensor that autograd saves inside the block (at least
    ``min_bytes`` large, on a CUDA device, not a parameter) for offload: the device→host copy runs on a side stream
    right away; in backward the first tensor of layer ``i`` that is needed triggers the host→device copies of layer
    ``i - prefetch`` as well, so they overlap the backward of the layers in between. On CPU tensors the hooks pass
    everything through, which is what the CPU tests exercise (bookkeeping and values)."""

    def __init__(self, prefetch: int = 1, min_bytes: int = 1 << 20):
        self.prefetch = max(int(prefetch), 0)
        self.min_bytes = min_bytes
        self.by_layer: Dict[int, List[_Handle]] = {}
        self.stream = None
        self.bytes_offloaded = 0
        self.param_ptrs = set()

    def _side(self, device):
        if self.stream is None:
            self.stream = torch.cuda.Stream(device=device)
        return self.stream

    def _pack(self, layer_id: int, t: torch.Tensor):
        if not t.is_cuda or t.numel() * t.element_size() < self.min_bytes or isinstance(t, torch.nn.Parameter) \
                or t.data_ptr() in self.param_ptrs:
            return t
        h = _Handle()
        h.layer, h.device, h.gpu, h.shape, h.dtype = layer_id, t.device, None, t.shape, t.dtype
        side = self._side(t.device)
        side.wait_stream(torch.cuda.current_stream(t.device))
        h.host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
        with torch.cuda.stream(side):
            h.host.copy_(t.contiguous(), non_blocking=True)
            h.event = torch.cuda.Event()
            h.event.record(side)
        t.record_stream(side)
        self.bytes_offloaded += t.numel() * t.element_size()
        self.by_layer.setdefault(layer_id, []).append(h)
        return h

    def _fetch(self, h: _Handle):
        if h.gpu is None and h.host is not None:
            side = self._side(h.device)
            with torch.cuda.stream(side):
                side.wait_event(h.event)
                h.gpu = torch.empty(h.shape, dtype=h.dtype, device=h.device)
                h.gpu.copy_(h.host, non_blocking=True)
                h.event = torch.cuda.Event()
                h.event.record(side)

    def _unpack(self, obj):
        if not isinstance(obj, _Handle):
            return obj
        for lid in (obj.layer, obj.layer - self.prefetch):
            for h in self.by_layer.get(lid, ()):
                self._fetch(h)
        torch.cuda.current_stream(obj.device).wait_event(obj.event)
        out = obj.gpu
        out.record_stream(torch.cuda.current_stream(obj.device))
        obj.gpu, obj.host = None, None
        return out

    def layer(self, layer_id: int):
        return torch.autograd.graph.saved_tensors_hooks(lambda t: self._pack(layer_id, t), self._unpack)

    def prune(self):
        """Drop the handles that backward has consumed (called when a new forward pass starts)."""
        for lid in list(self.by_layer):
            left = [h for h in self.by_layer[lid] if h.host is not None]
            if left:
                self.by_layer[lid] = left
            else:
                del self.by_layer[lid]

    def reset(self):
        """Call at the start of a step: handles of the previous step are released."""
        self.by_layer.clear()
        self.bytes_offloaded = 0
