"""Pre-LN transformer layer and the layer stack.

Reference: ``training_graph/transformer/transformer_layer.py`` (:74-250: input_layernorm →
self_attention → residual add → pre_mlp_layernorm → mlp → residual add, returning the extra (MoE) loss)
and ``transformer_block.py`` (:79-197: per-layer specs, final norm, loss threading), plus the layer →
pipeline-stage assignment with ``offset`` of ``training_graph/transformer/utils.py:93-159``.

The residual add of each sub-layer is folded into the following RMSNorm kernel: a layer receives the
pending sub-layer output and the residual stream and returns the same pair.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, List, Optional

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from .. import parallel_state as ps
from ..spec_utils import build_module
from .attention import AttnMeta
from .moe import MoELayer
from .norm import build_norm


@dataclass
class TransformerLayerSubmodules:
    """What a layer is made of, as ``ModuleSpec`` entries (``gpt_layer_specs.py`` fills them in). Norm entries are
    built with ``(config)``, the attention and an MoE ``mlp`` with ``(config, layer_number)``, a dense ``mlp`` with
    ``(config)``; ``None`` for a post-norm leaves it out."""
    input_layernorm: Any = None
    self_attention: Any = None
    pre_mlp_layernorm: Any = None
    mlp: Any = None
    post_attn_layernorm: Any = None
    post_mlp_layernorm: Any = None


class TransformerLayer(nn.Module):
    """Pre-LN block: ``input_layernorm`` → ``self_attention`` → ``pre_mlp_layernorm`` → ``mlp`` (dense or MoE), optional
    sandwich norms; the residual adds are folded into the norms. Built from a ``TransformerLayerSubmodules`` spec
    (reference ``training_graph/transformer/transformer_layer.py:74-250``)."""

    def __init__(self, config, layer_number: int = 1, is_moe: bool = False,
                 submodules: Optional[TransformerLayerSubmodules] = None):
        super().__init__()
        self.config = config
        self.layer_number = layer_number
        if submodules is None:     # the layer that the configuration describes
            from .gpt_layer_specs import get_gpt_layer_spec_for_config
            submodules = get_gpt_layer_spec_for_config(config, is_moe).submodules
        self.input_layernorm = build_module(submodules.input_layernorm, config)
        self.self_attention = build_module(submodules.self_attention, config, layer_number)
        self.pre_mlp_layernorm = build_module(submodules.pre_mlp_layernorm, config)
        mlp_spec = submodules.mlp
        mlp_cls = getattr(mlp_spec, "module", mlp_spec)
        self.is_moe = isinstance(mlp_cls, type) and issubclass(mlp_cls, MoELayer)
        self.mlp = build_module(mlp_spec, config, layer_number) if self.is_moe else build_module(mlp_spec, config)
        self.post_attn_layernorm = (build_module(submodules.post_attn_layernorm, config)
                                    if submodules.post_attn_layernorm is not None else None)
        self.post_mlp_layernorm = (build_module(submodules.post_mlp_layernorm, config)
                                   if submodules.post_mlp_layernorm is not None else None)
        self.hidden_dropout = float(getattr(config, "hidden_dropout", 0.0) or 0.0)

    def _dropout(self, x):
        """Hidden dropout on a sub-layer output before it joins the residual (reference ``bias_dropout_add``,
        ``transformer_layer.py:215-250``). Under sequence parallelism every tensor-parallel rank holds other tokens, so
        the mask comes from the tensor-parallel random stream (different per rank); otherwise the ranks hold the same
        activations and draw the same mask from the default stream."""
        if self.hidden_dropout <= 0.0 or not self.training:
            return x
        cfg = self.config
        if cfg.sequence_parallel and ps.get_tensor_model_parallel_world_size() > 1:
            from ...modules.rng import get_rng_tracker
            tracker = get_rng_tracker()
            if "model-parallel-rng" in tracker.states:
                with tracker.fork():
                    return torch.nn.functional.dropout(x, self.hidden_dropout, True)
        return torch.nn.functional.dropout(x, self.hidden_dropout, True)

    def forward(self, pending, residual, rotary, meta: AttnMeta):
        """``pending``: sub-layer output not yet added to ``residual`` (``residual`` None for the first layer)."""
        if residual is None:
            residual = pending
            normed = self.input_layernorm(pending)
        else:
            normed, residual = self.input_layernorm(pending, residual)
        attn_out, _ = self.self_attention(normed, rotary, meta)
        if self.post_attn_layernorm is not None:
            attn_out = self.post_attn_layernorm(attn_out)
        attn_out = self._dropout(attn_out)
        normed, residual = self.pre_mlp_layernorm(attn_out, residual)
        aux = None
        if self.is_moe:
            mlp_out, aux = self.mlp(normed)
        else:
            mlp_out, _ = self.mlp(normed)
        if self.post_mlp_layernorm is not None:
            mlp_out = self.post_mlp_layernorm(mlp_out)
        return self._dropout(mlp_out), residual, aux


def pipeline_layer_split(num_layers: int, pp: int, vpp: int = 1, offset=0) -> List[List[List[int]]]:
    """Layer ids of every (pp stage, virtual chunk). ``offset`` adds/removes layers per stage
    (list of pp values, or vpp lists of pp values), as the reference's ``LayerSetting`` does."""
    vpp = vpp or 1
    chunks = pp * vpp
    base = num_layers // chunks
    if isinstance(offset, int):
        if offset != 0:
            raise ValueError("a scalar offset must be 0; give a list with one value per stage")
        off = [[0] * pp for _ in range(vpp)]
    else:
        off = [list(o) for o in offset] if offset and isinstance(offset[0], (list, tuple)) else [list(offset)]
        if len(off) != vpp or any(len(o) != pp for o in off):
            raise ValueError(f"offset must hold {vpp} x {pp} values, got {offset!r}")
    counts = [[base + off[v][s] for s in range(pp)] for v in range(vpp)]
    if sum(sum(c) for c in counts) != num_layers:
        raise ValueError(f"layers per stage {counts} do not add up to num_layers={num_layers}")
    out = [[[] for _ in range(vpp)] for _ in range(pp)]
    nxt = 0
    for v in range(vpp):
        for s in range(pp):
            out[s][v] = list(range(nxt, nxt + counts[v][s]))
            nxt += counts[v][s]
    return out


class StageLayers(nn.Module):
    """The layers of one pipeline stage, registered under their GLOBAL layer number: a parameter of the sixth layer of
    the model is ``layers.5.…`` on whichever stage owns it, so checkpoints, weight loaders and resharding tools see
    one name space for every pipeline layout (the reference numbers layers globally per stage,
    ``training_graph/transformer/utils.py:129-159``). Iteration and integer indexing are over the stage's own
    layers in order (``layers[0]`` is the first layer of this stage), as with a ``ModuleList``."""

    def __init__(self, layer_ids, modules):
        super().__init__()
        self.layer_ids = list(layer_ids)
        for gid, mod in zip(self.layer_ids, modules):
            self.add_module(str(gid), mod)

    def __len__(self):
        return len(self.layer_ids)

    def __iter__(self):
        return (self._modules[str(g)] for g in self.layer_ids)

    def __getitem__(self, idx):
        if isinstance(idx, slice):
            return [self._modules[str(g)] for g in self.layer_ids[idx]]
        return self._modules[str(self.layer_ids[idx])]


class TransformerBlock(nn.Module):
    """The layers owned by this pipeline stage (and virtual chunk) plus, on the last stage, the final norm."""

    def __init__(self, config, pre_process: bool = True, post_process: bool = True, vp_stage: Optional[int] = None,
                 base_seed: Optional[int] = None):
        super().__init__()
        self.config = config
        base_seed = torch.initial_seed() if base_seed is None else base_seed
        dev = getattr(config, "device", None)
        pp = ps.get_pipeline_model_parallel_world_size()
        pp_rank = ps.get_pipeline_model_parallel_rank()
        vpp = config.virtual_pipeline_model_parallel_size or 1
        split = pipeline_layer_split(config.num_layers, pp, vpp, config.offset or 0)
        self.layer_ids = split[pp_rank][vp_stage or 0]
        from .gpt_layer_specs import get_gpt_decoder_block_spec
        layer_specs = get_gpt_decoder_block_spec(config)      # one spec per layer of the whole model
        from ..init_method import module_rng
        built = []
        for i in self.layer_ids:
            with module_rng(base_seed, 100 + i, dev):     # a layer's initial weights depend on its number only
                built.append(build_module(layer_specs[i], config, layer_number=i + 1))
        self.layers = StageLayers(self.layer_ids, built)
        self.final_layernorm = build_norm(config) if post_process else None
        self.recompute = bool(config.recompute) if not isinstance(config.recompute, (list, tuple)) else True
        self._recompute_layers = self._resolve_recompute(config.recompute)
        self._setup_selective_recompute_and_offload(config)
        # ``grads_final_hook(layer_id)``: set by the optimizer for the forward pass of a step's last micro-batch; it is
        # called during the backward pass as soon as every gradient of that layer's parameters has been written
        self.grads_final_hook = None
        # ``params_ready_hook(layer_id)``: set by the optimizer while it still publishes updated parameters; called
        # before a layer runs, it makes the stream wait for that layer's parameters
        self.params_ready_hook = None

    # reference defaults of ``select_recompute: true`` (``training_graph/transformer/utils.py:107-110``): the gated
    # activation of the MLP and of the shared experts; here these, the norms and the rotary embedding are what a
    # selectively recomputed layer runs twice, whatever the patterns say, because nothing else is cheap
    _DEFAULT_SELECT = (r"mlp\.mul", r"mlp\.activation_func\.silu", r"mlp\.shared_experts\.mul",
                       r"mlp\.shared_experts\.activation_func\.silu", r".*\.norm")

    def _setup_selective_recompute_and_offload(self, config):
        from ..recompute import ActivationOffloader, mark_recompute_modules
        n = len(self.layer_ids)
        sel = getattr(config, "select_recompute", False)
        patterns, count = [], 0
        if isinstance(sel, dict):                       # {pattern: layers per stage}
            patterns, count = list(sel.keys()), n
            counts = [self._resolve_recompute(v) for v in sel.values()]
            count = max(counts) if counts else 0
        elif isinstance(sel, (list, tuple)) and sel and all(isinstance(x, str) for x in sel):
            patterns, count = list(sel), n
        else:
            count = self._resolve_recompute(sel)
        self._select_layers = count
        extra = [p for p in patterns if p not in self._DEFAULT_SELECT]
        self._select_matched = []
        for layer in self.layers[:count]:
            self._select_matched += mark_recompute_modules(layer, extra)
        ignored = [k for k in ("recompute_slice_activation", "select_comm_recompute", "parallel_optimizer_comm_recompute")
                   if getattr(config, k, False)]
        if ignored:
            from ...tools.logger import logger
            logger.warning("recompute options without effect here: %s (the fused GEMM + collective kernels leave no "
                           "separate communication output to recompute, activations are not sliced)", ignored)
        # offload: ``swap: true`` with ``layer_swap`` = number of layers (or a list of {layers, backward_prefetch})
        self._offload = None
        self._offload_layers = set()
        if getattr(config, "cpu_offloading", False):
            spec = getattr(config, "cpu_offloading_num_layers", None)
            prefetch = int(getattr(config, "default_prefetch", 1) or 1)
            if isinstance(spec, (list, tuple)) and spec and isinstance(spec[0], dict):
                for entry in spec:
                    ids = entry.get("layers", True)
                    prefetch = int(entry.get("backward_prefetch", prefetch) or prefetch)
                    self._offload_layers |= set(range(n)) if ids is True else {int(i) for i in ids if int(i) < n}
            else:
                k = n if spec in (None, True) else min(int(spec), n)
                self._offload_layers = set(range(k))
            self._offload = ActivationOffloader(prefetch=prefetch)

    def _resolve_recompute(self, rc):
        n = len(self.layer_ids)
        if isinstance(rc, bool):
            return n if rc else 0
        if isinstance(rc, int):
            return min(rc, n)
        if isinstance(rc, (list, tuple)) and rc:
            pp_rank = ps.get_pipeline_model_parallel_rank()
            val = rc[pp_rank] if pp_rank < len(rc) else rc[-1]
            if isinstance(val, (list, tuple)):
                val = val[0]
            return n if val is True else int(val or 0)
        return 0

    def forward(self, hidden, rotary, meta: AttnMeta):
        pending, residual = hidden, None
        aux_total = None
        training = self.training and torch.is_grad_enabled()
        if training and self._offload is not None:
            self._offload.prune()
        for idx, layer in enumerate(self.layers):
            run = layer
            if self.params_ready_hook is not None:
                self.params_ready_hook(self.layer_ids[idx])
            if training and self.grads_final_hook is not None and pending.requires_grad:
                # the gradient of a layer's input is the last thing its backward pass produces
                def fire(_grad, _cb=self.grads_final_hook, _gid=self.layer_ids[idx]):
                    _cb(_gid)
                pending.register_hook(fire)
            if training and self._offload is not None and idx in self._offload_layers:
                def run(p, r, ro, m, _layer=layer, _idx=idx):     # saved tensors of this layer go to pinned host memory
                    with self._offload.layer(_idx):
                        return _layer(p, r, ro, m)
            if training and idx < self._recompute_layers:
                pending, residual, aux = checkpoint(run, pending, residual, rotary, meta, use_reentrant=False)
            elif training and idx < self._select_layers:
                from ..recompute import selective_checkpoint
                pending, residual, aux = selective_checkpoint(run, pending, residual, rotary, meta)
            else:
                pending, residual, aux = run(pending, residual, rotary, meta)
            if aux is not None:
                aux_total = aux if aux_total is None else aux_total + aux
        if self.final_layernorm is not None:
            if residual is None:
                out = self.final_layernorm(pending)
            else:
                out, _ = self.final_layernorm(pending, residual)
        else:
            out = pending if residual is None else pending + residual
        return out, aux_total
