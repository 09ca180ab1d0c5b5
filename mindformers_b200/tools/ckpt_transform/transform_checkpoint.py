"""``TransformCkpt``: rewrite a checkpoint saved under one parallel layout as the per-rank files of another.

Reference: ``tools/ckpt_transform/transform_checkpoint.py`` (``TransformCkpt`` :57, ``__call__`` :168,
``transform_ckpt`` :287): source strategy + destination strategy → unify → re-slice, one output directory
``rank_N`` per destination rank. Here the strategies are the JSON files that ``checkpoint/sharding.py::save_strategy``
writes next to every run's checkpoints (``ckpt_strategy_rank_N.json``: per parameter its shape and tensor- / expert-
parallel slicing). A destination strategy is produced by starting the destination job with ``only_save_strategy: true``
(or by ``save_strategy`` on its model).

    python -m mindformers_b200.tools.transform_ckpt --src_ckpt_dir output/checkpoint --src_ckpt_strategy output/strategy \\
        --dst_ckpt_strategy new_layout/strategy --dst_ckpt_dir transformed --prefix llama

Optimizer moments (``adam_m.*`` / ``adam_v.*``) follow their parameter's slicing; a destination job with a sharded
optimizer cuts its data-parallel slice out of them when it loads.
"""
from __future__ import annotations

import glob
import json
import os
import shutil
import tempfile
from typing import Dict, Optional

import torch
from safetensors.torch import load_file, save_file

from ...checkpoint.transform import _STATE_PREFIXES, unify_checkpoints
from ...parallel.layers.tensor_parallel import shard_sections
from ...tools.logger import logger


def slice_for_layout(full: torch.Tensor, layout: dict) -> torch.Tensor:
    """The part of a full tensor that the rank described by ``layout`` holds (``layout["shape"]`` is that part's shape)."""
    t = full
    if layout.get("ep", 1) > 1:
        per = t.shape[0] // layout["ep"]
        t = t[layout["ep_rank"] * per:(layout["ep_rank"] + 1) * per]
    tp, dim = layout.get("tp", 1), layout.get("dim", -1)
    if tp > 1 and dim >= 0:
        rank = layout["tp_rank"]
        if layout.get("sections"):
            t = shard_sections(t, layout["sections"], dim, rank, tp, layout.get("groups"))
        else:
            per = int(layout["shape"][dim])
            if per * tp != t.shape[dim]:                  # padded vocabulary
                shape = list(t.shape)
                shape[dim] = per * tp - t.shape[dim]
                t = torch.cat((t, t.new_zeros(shape)), dim=dim)
            t = t.narrow(dim, rank * per, per)
    if list(t.shape) != [int(x) for x in layout["shape"]]:
        raise ValueError(f"tensor of shape {tuple(full.shape)} does not give the slice {layout['shape']} of the destination")
    return t.contiguous()


class TransformCkpt:
    """``TransformCkpt()(src_checkpoint, dst_checkpoint_dir, src_strategy, dst_strategy, prefix)``.

    ``src_checkpoint``: a directory with ``rank_N`` sub-directories (with ``src_strategy``: the directory of their
    strategy files) or an already complete checkpoint (a ``.safetensors`` file or a directory of them; no
    ``src_strategy``). ``dst_strategy``: directory of the destination layout's ``ckpt_strategy_rank_N.json`` files;
    None writes the complete checkpoint. Returns ``dst_checkpoint_dir``."""

    def __init__(self, include_optimizer: bool = True, rank_id: Optional[int] = None, world_size: Optional[int] = None, **kwargs):
        self.include_optimizer = include_optimizer
        self.rank_id, self.world_size = rank_id, world_size

    @staticmethod
    def _load_full(path: str) -> Dict[str, torch.Tensor]:
        files = [path] if os.path.isfile(path) else sorted(glob.glob(os.path.join(path, "*.safetensors")))
        if not files:
            raise FileNotFoundError(f"no safetensors file in {path}")
        out: Dict[str, torch.Tensor] = {}
        for f in files:
            out.update(load_file(f))
        return out

    def __call__(self, src_checkpoint: str, dst_checkpoint_dir: str, src_strategy: Optional[str] = None,
                 dst_strategy: Optional[str] = None, prefix: str = "checkpoint_") -> str:
        tmp = None
        try:
            if src_strategy:
                tmp = tempfile.mkdtemp(prefix="unified_")
                unify_checkpoints(src_checkpoint, src_strategy, tmp, include_optimizer=self.include_optimizer)
                full = self._load_full(tmp)
            else:
                full = self._load_full(src_checkpoint)
            os.makedirs(dst_checkpoint_dir, exist_ok=True)
            if not dst_strategy:
                model = {k: v for k, v in full.items() if not k.startswith(_STATE_PREFIXES) and v.dim() > 0}
                rest = {k: v for k, v in full.items() if k not in model}
                save_file({k: v.contiguous() for k, v in model.items()}, os.path.join(dst_checkpoint_dir, "model.safetensors"),
                          metadata={"format": "pt"})
                if rest and self.include_optimizer:
                    save_file({k: v.contiguous() for k, v in rest.items()},
                              os.path.join(dst_checkpoint_dir, "hyper_param.safetensors"), metadata={"format": "pt"})
                return dst_checkpoint_dir
            files = sorted(glob.glob(os.path.join(dst_strategy, "ckpt_strategy_rank_*.json")),
                           key=lambda f: int(os.path.basename(f).split("_")[-1].split(".")[0]))
            if not files:
                raise FileNotFoundError(f"no ckpt_strategy_rank_N.json in {dst_strategy}")
            scalars = {k: v for k, v in full.items() if v.dim() == 0}
            for f in files:
                rank = int(os.path.basename(f).split("_")[-1].split(".")[0])
                if self.rank_id is not None and self.world_size and rank % self.world_size != self.rank_id:
                    continue                                   # several processes share the destination ranks
                with open(f) as fh:
                    params = json.load(fh)["params"]
                out: Dict[str, torch.Tensor] = {}
                for name, lay in params.items():
                    if name not in full:
                        raise KeyError(f"{name} (rank {rank} of the destination) is not in the source checkpoint")
                    out[name] = slice_for_layout(full[name], lay)
                    if self.include_optimizer:
                        for pre in _STATE_PREFIXES:
                            if pre + name in full and full[pre + name].shape == full[name].shape:
                                out[pre + name] = slice_for_layout(full[pre + name], lay)
                if self.include_optimizer:
                    out.update(scalars)
                rank_dir = os.path.join(dst_checkpoint_dir, f"rank_{rank}")
                os.makedirs(rank_dir, exist_ok=True)
                save_file(out, os.path.join(rank_dir, f"{prefix}rank_{rank}.safetensors"), metadata={"format": "pt"})
                logger.info("transformed checkpoint of rank %d: %d tensors", rank, len(out))
            return dst_checkpoint_dir
        finally:
            if tmp:
                shutil.rmtree(tmp, ignore_errors=True)
