"""Streaming weight loading: lazy slices of safetensors files, tensor-parallel splits, layer-by-layer conversion.

Reference: ``parallel_core/inference/weights_utils.py`` (``WeightsLoader:28`` with lazy ``safe_open`` slices,
``split_by_tp_rank_rows / columns``, QKV / FFN concatenation with KV-head replication, expert stacking, the MLA
rope-dimension de-interleave ``infer_trans_rope_weight:244-249``) and ``base_models/gpt/gpt_model.py`` ``load_weights``
(streams a Hugging Face or framework checkpoint layer by layer).

``checkpoint/io.py::load_checkpoint`` reads whole files, which is fine for training checkpoints of this rank. A
pretrained directory of hundreds of GB is loaded here instead: the loader indexes which file holds which tensor
(``*.index.json`` or the file headers), and ``load_weights`` walks the checkpoint one transformer layer at a time —
read the layer's tensors, convert names and fused layouts with the same code as the offline converter
(``checkpoint/name_maps.py``), copy this rank's shard into the parameters, drop the layer — so the host never holds
more than one layer. Row- or column-sharded tensors that need no fusing (embedding, output head) are read as slices.
"""
from __future__ import annotations

import glob
import json
import os
import re
from typing import Dict, Iterable, List, Tuple

import torch
from safetensors import safe_open

from ..checkpoint import name_maps
from ..checkpoint.sharding import shard_for_param
from ..tools.logger import logger

_LAYER_RE = re.compile(r"^(?:model\.|transformer\.encoder\.)?(?:decoder\.)?layers\.(\d+)\.")


def split_by_tp_rank_rows(sl, rank: int, world: int) -> torch.Tensor:
    """Rows ``[rank * n / world, (rank + 1) * n / world)`` of a lazy slice (or tensor)."""
    n = sl.get_shape()[0] if hasattr(sl, "get_shape") else sl.shape[0]
    if n % world:
        raise ValueError(f"{n} rows do not split over {world} ranks")
    per = n // world
    return sl[rank * per:(rank + 1) * per]


def split_by_tp_rank_columns(sl, rank: int, world: int) -> torch.Tensor:
    shape = sl.get_shape() if hasattr(sl, "get_shape") else sl.shape
    n = shape[1]
    if n % world:
        raise ValueError(f"{n} columns do not split over {world} ranks")
    per = n // world
    return sl[:, rank * per:(rank + 1) * per]


def infer_trans_rope_weight(weight: torch.Tensor, rope_dim: int) -> torch.Tensor:
    """The last ``rope_dim`` rows of every head block reordered from interleaved pairs ``(x0, y0, x1, y1, ..)`` to
    halves ``(x0, x1, .., y0, y1, ..)``: checkpoints trained with interleaved RoPE served by a rotate-half kernel."""
    w = weight.clone()
    rope = w[-rope_dim:]
    w[-rope_dim:] = torch.cat((rope[0::2], rope[1::2]), dim=0)
    return w


class WeightsLoader:
    """Index of a directory (or list) of safetensors files with lazy access to single tensors and slices."""

    def __init__(self, path):
        if isinstance(path, (list, tuple)):
            files = list(path)
            root = os.path.dirname(files[0]) if files else "."
        elif os.path.isdir(path):
            root, files = path, sorted(glob.glob(os.path.join(path, "*.safetensors")))
        else:
            root, files = os.path.dirname(path), [path]
        if not files:
            raise FileNotFoundError(f"no safetensors files under {path}")
        self.root, self.files = root, files
        self.key_to_file: Dict[str, str] = {}
        index = glob.glob(os.path.join(root, "*.safetensors.index.json"))
        if index and os.path.isdir(str(path)):
            with open(index[0]) as f:
                for k, fn in json.load(f).get("weight_map", {}).items():
                    self.key_to_file[k] = os.path.join(root, fn)
        else:
            for fn in files:
                with safe_open(fn, framework="pt") as f:
                    for k in f.keys():
                        self.key_to_file[k] = fn
        self._open: Dict[str, object] = {}

    # ---- access ---------------------------------------------------------------------------------------------
    def _handle(self, fn: str):
        h = self._open.get(fn)
        if h is None:
            h = self._open[fn] = safe_open(fn, framework="pt")
        return h

    def keys(self) -> List[str]:
        return list(self.key_to_file)

    def has(self, name: str) -> bool:
        return name in self.key_to_file

    def get_slice(self, name: str):
        """Lazy view: index it (``sl[a:b]``, ``sl[:, a:b]``) to read just those rows / columns from disk."""
        return self._handle(self.key_to_file[name]).get_slice(name)

    def get(self, name: str) -> torch.Tensor:
        return self._handle(self.key_to_file[name]).get_tensor(name)

    def shape(self, name: str) -> Tuple[int, ...]:
        return tuple(self.get_slice(name).get_shape())

    def rows(self, name: str, rank: int, world: int) -> torch.Tensor:
        return split_by_tp_rank_rows(self.get_slice(name), rank, world)

    def columns(self, name: str, rank: int, world: int) -> torch.Tensor:
        return split_by_tp_rank_columns(self.get_slice(name), rank, world)

    def load_group(self, names: Iterable[str]) -> Dict[str, torch.Tensor]:
        return {n: self.get(n) for n in names}

    def close(self):
        self._open.clear()

    # ---- grouping -------------------------------------------------------------------------------------------
    def layer_groups(self) -> Tuple[Dict[int, List[str]], List[str]]:
        """``({layer index: keys}, keys outside the layers)``."""
        layers: Dict[int, List[str]] = {}
        other: List[str] = []
        for k in self.key_to_file:
            m = _LAYER_RE.match(k)
            if m:
                layers.setdefault(int(m.group(1)), []).append(k)
            else:
                other.append(k)
        return layers, other


def _assign(model, params, buffers, fw: Dict[str, torch.Tensor], used: set, fp8_modules: list, keep_fp8: bool):
    from ..checkpoint.io import _owner_path
    with torch.no_grad():
        for n, t in fw.items():
            if n.endswith("_scale_inv"):
                continue
            p = params.get(n)
            if p is None:
                b = buffers.get(n)
                if b is not None and tuple(b.shape) == tuple(t.shape):
                    b.copy_(t.to(device=b.device, dtype=b.dtype))
                    used.add(n)
                continue
            if t.dtype == torch.float8_e4m3fn:
                t = name_maps.weight_dequant(t, fw[n + "_scale_inv"])
                owner = model.get_submodule(_owner_path(model, n))
                if keep_fp8 and hasattr(owner, "quantize_fp8_"):
                    fp8_modules.append(owner)
            p.copy_(shard_for_param(t, p).to(device=p.device, dtype=p.dtype))
            used.add(n)


def load_weights(model: torch.nn.Module, path: str, family: str = "llama", strict: bool = True,
                 keep_fp8: bool = False) -> dict:
    """Stream a Hugging Face style (or framework-named) safetensors directory into ``model``, one layer at a time.

    Returns ``{"layers": n, "tensors": n, "peak_group_bytes": n, "missing": [...]}``. ``keep_fp8`` re-quantises the
    local shards of layers that arrived as block-scaled fp8 (``Column/RowParallelLinear.quantize_fp8_``)."""
    loader = WeightsLoader(path)
    layers, other = loader.layer_groups()
    params = dict(model.named_parameters())
    buffers = dict(model.named_buffers())
    is_hf = any(k.startswith(("model.", "lm_head", "transformer.")) for k in loader.keys())
    used: set = set()
    fp8_modules: list = []
    peak = 0
    groups = [sorted(other)] + [sorted(layers[i]) for i in sorted(layers)]
    for names in groups:
        if not names:
            continue
        part = loader.load_group(names)
        peak = max(peak, sum(t.numel() * t.element_size() for t in part.values()))
        fw = name_maps.hf_to_framework(part, model.config, family, keep_fp8=keep_fp8) if is_hf else part
        _assign(model, params, buffers, fw, used, fp8_modules, keep_fp8)
        del part, fw
    if "output_layer.weight" in params and "output_layer.weight" not in used \
            and not getattr(model.config, "untie_embeddings_and_output_weights", True) \
            and "embedding.word_embeddings.weight" in used:
        with torch.no_grad():
            params["output_layer.weight"].copy_(params["embedding.word_embeddings.weight"])
        used.add("output_layer.weight")
    for mod in fp8_modules:
        mod.quantize_fp8_()
    loader.close()
    missing = [n for n in params if n not in used]
    if missing and strict:
        raise KeyError(f"{path} lacks parameters: {missing[:8]}{' ...' if len(missing) > 8 else ''}")
    if missing:
        logger.warning("parameters not found in %s: %s", path, missing[:8])
    return {"layers": len(layers), "tensors": len(loader.key_to_file), "peak_group_bytes": peak, "missing": missing}


def split_weight_by_tp_rank(weight, split_axis: int, tp_rank_id: int, tp_group_size: int) -> torch.Tensor:
    """This rank's equal share of ``weight`` (a tensor or a lazy safetensors slice) along ``split_axis`` (0 = rows,
    1 = columns); reference ``parallel_core/inference/weights_utils.py:252``."""
    if split_axis == 0:
        return split_by_tp_rank_rows(weight, tp_rank_id, tp_group_size)
    if split_axis == 1:
        return split_by_tp_rank_columns(weight, tp_rank_id, tp_group_size)
    raise ValueError(f"split_axis must be 0 or 1, got {split_axis}")


def handle_training_ffn_weight(ffn_value: torch.Tensor):
    """Packed ``[gate; up]`` first projection of a training checkpoint → ``(gate, up)`` halves along the rows."""
    gate, up = ffn_value.chunk(2, dim=0)
    return gate.contiguous(), up.contiguous()


def handle_training_qkv_weight(qkv_weight_value: torch.Tensor, config):
    """Group-interleaved packed QKV of a training checkpoint (per KV group: its ``heads / groups`` query heads, then its
    key, then its value) → ``(q, k, v)`` in head order."""
    heads = config.num_attention_heads
    groups = getattr(config, "num_query_groups", None) or heads
    hd = getattr(config, "kv_channels", None) or config.hidden_size // heads
    rep = heads // groups
    w = qkv_weight_value.reshape(groups, (rep + 2) * hd, -1)
    q = w[:, : rep * hd].reshape(heads * hd, -1)
    k = w[:, rep * hd: (rep + 1) * hd].reshape(groups * hd, -1)
    v = w[:, (rep + 1) * hd:].reshape(groups * hd, -1)
    return q.contiguous(), k.contiguous(), v.contiguous()
