"""Checkpoint save / load in safetensors with the reference's directory scheme.

Save layout (reference ``core/callback/callback.py:1203-1645``):
``<dir>/rank_{r}/{prefix}_rank_{r}-{epoch}_{step}.safetensors`` + ``meta.json`` (last file, epoch, step) in the
same rank directory; network-only copies under ``checkpoint_network``; a JSON strategy file per rank under
``strategy/``. Saved state: model parameters, optimizer moments ``adam_m.*`` / ``adam_v.*`` (and the 16-bit fp32
master remainders ``master_lo.*``), plus ``global_step, epoch_num, step_num, loss_scale, global_batch_size``
as 0-d tensors (reference ``callback.py:1397-1411``).

Load accepts the three layouts of ``utils/load_checkpoint_utils.py:100-122`` (single file, directory of files,
``rank_N`` directories) and Hugging Face model directories (``config.json`` + ``*.safetensors``), which are
renamed and fused on the fly and then sliced for this rank.
"""
from __future__ import annotations

import glob
import json
import os
import shutil
from typing import Dict, Optional, Tuple

import torch
from safetensors import safe_open
from safetensors.torch import load_file, save_file

from ..parallel import parallel_state as ps
from ..tools.logger import logger
from ..tools.utils import format_ckpt_name, get_real_rank, parse_ckpt_name
from . import name_maps
from .sharding import save_strategy, shard_for_param

TRANSIENT_KEYS = ("accu_grads", "key_cache", "value_cache", "expert_load", "rotary_pos_emb")
SCALAR_KEYS = ("global_step", "epoch_num", "step_num", "loss_scale", "global_batch_size")


def _is_transient(name: str) -> bool:
    return any(k in name for k in TRANSIENT_KEYS)


def _sync_params(model):
    """An optimizer that still publishes updated parameters on a side stream leaves a hook on the model: wait for it."""
    fn = getattr(model, "_mfb_param_sync", None)
    if callable(fn):
        fn()


def model_state(model: torch.nn.Module, trainable_only: bool = False) -> Dict[str, torch.Tensor]:
    _sync_params(model)
    out = {}
    for n, p in model.named_parameters():
        if trainable_only and not p.requires_grad:
            continue
        out[n] = p.detach()
    for n, b in model.named_buffers():
        if not _is_transient(n) and b is not None and n.split(".")[-1] in ("expert_bias",):
            out[n] = b.detach()
    return out


def _to_host(t: torch.Tensor) -> torch.Tensor:
    """A host copy that no later device work can change. CUDA tensors are copied into pinned memory on the current
    stream (the caller synchronises once after all copies are queued)."""
    t = t.detach()
    if t.is_cuda:
        host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
        host.copy_(t, non_blocking=True)
        return host
    return t.contiguous().clone()


def snapshot_checkpoint(model: torch.nn.Module, *, optimizer=None, epoch: int = 0, step: int = 0,
                        extra: Optional[dict] = None, trainable_only: bool = False,
                        remove_redundancy: bool = False) -> Dict[str, torch.Tensor]:
    """Host snapshot of everything a checkpoint file holds, taken on the training stream: parameters, this rank's
    optimizer states and the scalar entries. After this returns the training loop may go on changing the device
    tensors; ``write_checkpoint`` (possibly on another thread) only sees the copies."""
    tensors: Dict[str, torch.Tensor] = {}
    for n, t in model_state(model, trainable_only).items():
        if remove_redundancy and _is_redundant(n, model):
            continue
        tensors[n] = _to_host(t)
    if optimizer is not None and hasattr(optimizer, "named_states"):
        for n, t in optimizer.named_states().items():
            tensors[n] = _to_host(t)
        tensors["global_step"] = torch.tensor(int(getattr(optimizer, "global_step", 0)), dtype=torch.int64)
    if torch.cuda.is_available():
        torch.cuda.current_stream().synchronize()
    scalars = {"epoch_num": epoch, "step_num": step}
    scalars.update(extra or {})
    for k, v in scalars.items():
        tensors[k] = torch.tensor(v, dtype=torch.float32 if isinstance(v, float) else torch.int64)
    return tensors


def write_checkpoint(tensors: Dict[str, torch.Tensor], directory: str, *, rank: Optional[int] = None,
                     prefix: str = "mindformers", epoch: int = 0, step: int = 0, keep_max: int = 5,
                     remove_redundancy: bool = False, network_only_dir: Optional[str] = None) -> str:
    """Write a snapshot as ``rank_{r}/{prefix}_rank_{r}-{epoch}_{step}.safetensors`` (atomically), update
    ``meta.json`` and rotate old files. Touches no device memory: safe on a background thread."""
    rank = get_real_rank() if rank is None else rank
    rank_dir = os.path.join(directory, f"rank_{rank}")
    os.makedirs(rank_dir, exist_ok=True)
    name = format_ckpt_name(prefix, rank, epoch, step)
    path = os.path.join(rank_dir, name)
    tmp = path + ".tmp"
    save_file(tensors, tmp, metadata={"format": "pt", "remove_redundancy": str(bool(remove_redundancy))})
    os.replace(tmp, path)
    meta = {"last_epoch": epoch, "last_step": step, "last_ckpt_file": name}
    mtmp = os.path.join(rank_dir, "meta.json.tmp")
    with open(mtmp, "w") as f:
        json.dump(meta, f)
    os.replace(mtmp, os.path.join(rank_dir, "meta.json"))
    _rotate(rank_dir, prefix, keep_max)
    if network_only_dir:
        ndir = os.path.join(network_only_dir, f"rank_{rank}")
        os.makedirs(ndir, exist_ok=True)
        skip = ("adam_m.", "adam_v.", "master_lo.", "__slice__.")
        save_file({n: t for n, t in tensors.items() if not n.startswith(skip) and n not in SCALAR_KEYS},
                  os.path.join(ndir, name))
    return path


def save_checkpoint(model: torch.nn.Module, directory: str, *, optimizer=None, prefix: str = "mindformers",
                    epoch: int = 0, step: int = 0, extra: Optional[dict] = None, keep_max: int = 5,
                    save_network_only_copy: bool = False, trainable_only: bool = False,
                    remove_redundancy: bool = False, write_strategy: bool = True) -> str:
    """Write this rank's checkpoint (snapshot + write in one call); returns the file path."""
    tensors = snapshot_checkpoint(model, optimizer=optimizer, epoch=epoch, step=step, extra=extra,
                                  trainable_only=trainable_only, remove_redundancy=remove_redundancy)
    rank = get_real_rank()
    root = os.path.dirname(directory.rstrip("/")) or "."
    if write_strategy:
        save_strategy(model, os.path.join(root, "strategy", f"ckpt_strategy_rank_{rank}.json"))
    return write_checkpoint(tensors, directory, rank=rank, prefix=prefix, epoch=epoch, step=step, keep_max=keep_max,
                            remove_redundancy=remove_redundancy,
                            network_only_dir=os.path.join(root, "checkpoint_network") if save_network_only_copy else None)


def _is_redundant(name: str, model) -> bool:
    """A tensor-parallel-replicated parameter is written only by the first rank of its TP group."""
    p = dict(model.named_parameters()).get(name)
    if p is None:
        return False
    replicated = not getattr(p, "tensor_model_parallel", False) and not getattr(p, "is_expert", False)
    return replicated and ps.get_tensor_model_parallel_rank() != 0


def _rotate(rank_dir: str, prefix: str, keep_max: int):
    if keep_max is None or keep_max <= 0:
        return
    files = []
    for f in os.listdir(rank_dir):
        parsed = parse_ckpt_name(f)
        if parsed and parsed[0] == prefix:
            files.append(((parsed[2], parsed[3]), f))
    files.sort()
    for _, f in files[:-keep_max]:
        os.remove(os.path.join(rank_dir, f))


# --------------------------------------------------------------------------------------------------
def is_hf_safetensors_dir(path: str) -> bool:
    return os.path.isdir(path) and os.path.exists(os.path.join(path, "config.json")) and \
        bool(glob.glob(os.path.join(path, "*.safetensors")))


def _read_files(files) -> Dict[str, torch.Tensor]:
    out = {}
    for f in files:
        out.update(load_file(f))
    return out


def resolve_checkpoint(path: str, rank: Optional[int] = None, point: Optional[Tuple[int, int]] = None) -> Tuple[str, list]:
    """Classify ``path`` → (kind, files) with kind in {"file", "dir", "rank_dirs", "hf"}. With ``point`` =
    (epoch, step) the file of exactly that save is taken from the rank directory (the resume point that all ranks
    agreed on) instead of the rank's own newest file."""
    rank = get_real_rank() if rank is None else rank
    if os.path.isfile(path):
        return "file", [path]
    if is_hf_safetensors_dir(path):
        return "hf", sorted(glob.glob(os.path.join(path, "*.safetensors")))
    rdir = os.path.join(path, f"rank_{rank}")
    if os.path.isdir(rdir) and point is not None:
        from .resume import checkpoint_file_for
        f = checkpoint_file_for(path, rank, int(point[0]), int(point[1]))
        if f is None:
            raise FileNotFoundError(f"rank {rank} has no checkpoint of epoch {point[0]} step {point[1]} under {path}")
        return "rank_dirs", [f]
    if os.path.isdir(rdir):
        meta = os.path.join(rdir, "meta.json")
        if os.path.exists(meta):
            with open(meta) as f:
                last = json.load(f).get("last_ckpt_file")
            if last and os.path.exists(os.path.join(rdir, last)):
                return "rank_dirs", [os.path.join(rdir, last)]
        files = sorted(glob.glob(os.path.join(rdir, "*.safetensors")), key=lambda f: parse_ckpt_name(f)[2:] if parse_ckpt_name(f) else (0, 0))
        return "rank_dirs", files[-1:]
    files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
    if files:
        return "dir", files
    raise FileNotFoundError(f"no safetensors checkpoint found under {path}")


def _file_removed_redundancy(path: str) -> bool:
    try:
        with safe_open(path, framework="pt") as f:
            return (f.metadata() or {}).get("remove_redundancy") == "True"
    except Exception:  # noqa: BLE001  (an unreadable header shows up as a load error right after)
        return False


def _tp_first_rank_file(path: str, own_file: str) -> Optional[str]:
    """The file of the same save written by the first rank of this rank's tensor-parallel group (same data- and
    pipeline-parallel position): with ``remove_redundancy`` it alone holds the tensor-parallel-replicated tensors."""
    parsed = parse_ckpt_name(own_file)
    if parsed is None or not ps.model_parallel_is_initialized():
        return None
    first = ps.get_group_ranks("tp")[0]
    from .resume import checkpoint_file_for
    return checkpoint_file_for(path, first, parsed[2], parsed[3])


def load_checkpoint(model: torch.nn.Module, path: str, *, optimizer=None, strict: bool = True, family: str = "llama",
                    sharded: Optional[bool] = None, point: Optional[Tuple[int, int]] = None) -> dict:
    """Load parameters (and optimizer state when given). Returns the scalar entries (epoch, step, ...).

    ``sharded``: the tensors in the file are already this rank's slices (default for ``rank_N`` layouts); full
    tensors (single files, plain directories, HF directories) are sliced by ``shard_for_param``. ``point``: the
    (epoch, step) every rank resumes from (``checkpoint.resume.get_resume_checkpoint``).
    """
    kind, files = resolve_checkpoint(path, point=point)
    if kind == "hf" and optimizer is None:
        # a pretrained directory can be far larger than host memory: stream it layer by layer
        from ..inference.weights_utils import load_weights
        load_weights(model, path, family=family, strict=strict)
        return {}
    sd = _read_files(files)
    if kind == "rank_dirs" and files and _file_removed_redundancy(files[0]) and ps.get_tensor_model_parallel_rank() != 0:
        # replicated tensors were written by the first tensor-parallel rank only: take them from its file
        other = _tp_first_rank_file(path, files[0])
        if other is None:
            raise FileNotFoundError(f"{files[0]} was saved with remove_redundancy; the file of the first "
                                    "tensor-parallel rank, which holds the replicated tensors, is missing")
        extra_sd = load_file(other)
        own_params = dict(model.named_parameters())
        for k, v in extra_sd.items():
            base = k.split(".", 1)[1] if k.startswith(("adam_m.", "adam_v.", "master_lo.", "__slice__.")) else k
            p = own_params.get(base)
            replicated = p is not None and not getattr(p, "tensor_model_parallel", False) and not getattr(p, "is_expert", False)
            if k not in sd and replicated:
                sd[k] = v
    if kind == "hf":
        sd = name_maps.hf_to_framework(sd, model.config, family)
    elif any(name_maps.is_legacy_llama_name(k) for k in sd):
        # a checkpoint written by the reference's legacy Llama (model.layers.N.attention.wq ...): keep the scalars
        legacy = {k: v for k, v in sd.items() if k.startswith(("model.", "lm_head."))}
        rest = {k: v for k, v in sd.items() if k not in legacy}
        sd = dict(rest, **name_maps.legacy_llama_to_framework(legacy, model.config))
    if kind == "dir" and os.path.exists(os.path.join(path, "hyper_param.safetensors")) and "global_step" not in sd:
        sd.update(load_file(os.path.join(path, "hyper_param.safetensors")))
    if sharded is None:
        sharded = kind == "rank_dirs"
    params = dict(model.named_parameters())
    buffers = dict(model.named_buffers())
    missing, used = [], set()
    fp8_modules = []
    with torch.no_grad():
        for n, p in params.items():
            src = sd.get(n)
            if src is not None and src.dtype == torch.float8_e4m3fn:
                # block-scaled fp8 weight: de-quantise, load (and shard) like any other tensor, then re-quantise the
                # local shard in place once everything is loaded (shard boundaries are multiples of the 128 block)
                scale = sd.get(n + "_scale_inv")
                if scale is None:
                    raise KeyError(f"{n} is fp8 but {n}_scale_inv is missing from {path}")
                src = name_maps.weight_dequant(src, scale)
                used.add(n + "_scale_inv")
                owner = model.get_submodule(_owner_path(model, n))
                if hasattr(owner, "quantize_fp8_"):
                    fp8_modules.append(owner)
            if src is None and n == "output_layer.weight" and "embedding.word_embeddings.weight" in sd \
                    and not getattr(model.config, "untie_embeddings_and_output_weights", True):
                src = sd["embedding.word_embeddings.weight"]
            if src is None:
                missing.append(n)
                continue
            used.add(n)
            t = src if sharded and tuple(src.shape) == tuple(p.shape) else shard_for_param(src, p)
            p.copy_(t.to(device=p.device, dtype=p.dtype))
        for n, b in buffers.items():
            if n in sd and tuple(sd[n].shape) == tuple(b.shape):
                b.copy_(sd[n].to(device=b.device, dtype=b.dtype))
                used.add(n)
        for mod in fp8_modules:
            mod.quantize_fp8_()
    if missing and strict:
        raise KeyError(f"checkpoint {path} lacks parameters: {missing[:8]}{' ...' if len(missing) > 8 else ''}")
    if missing:
        logger.warning("parameters not found in checkpoint: %s", missing[:8])
    scalars = {k: sd[k].item() for k in SCALAR_KEYS if k in sd}
    if optimizer is not None:
        if hasattr(optimizer, "reload_model_params"):
            optimizer.reload_model_params()
        states = {k: v for k, v in sd.items() if k.startswith(("adam_m.", "adam_v.", "master_lo.", "__slice__."))}
        if states and hasattr(optimizer, "load_named_states"):
            optimizer.load_named_states(states, scalars.get("global_step"), strict=strict, model_params=params)
        elif "global_step" in scalars:
            optimizer.global_step = int(scalars["global_step"])
    return scalars


def _owner_path(model: torch.nn.Module, param_name: str) -> str:
    """Module path of a parameter name as ``named_parameters`` of the model reports it (wrappers that strip a
    ``model.`` prefix from their parameter names are looked through)."""
    mod_path = param_name.rsplit(".", 1)[0] if "." in param_name else ""
    try:
        model.get_submodule(mod_path)
        return mod_path
    except AttributeError:
        return "model." + mod_path if mod_path else "model"


def shard_checkpoint(state_dict: Dict[str, torch.Tensor], max_shard_size=5 << 30, weights_name: str = "model.safetensors"):
    """Cut a state dict into files of at most ``max_shard_size`` bytes, walking the keys in order (no bin packing; a
    tensor larger than the limit gets a file of its own). Returns ``(shards, index)``: ``{file name: {key: tensor}}`` and
    ``{"metadata": {"total_size"}, "weight_map": {key: file name}}`` — ``index`` is ``None`` for a single file, which
    then carries ``weights_name`` (reference ``models/modeling_utils.py:87-155``)."""
    limit = max_shard_size if isinstance(max_shard_size, int) else _size_to_int(max_shard_size)
    groups, cur, size, total = [], {}, 0, 0
    for n, t in state_dict.items():
        b = t.numel() * t.element_size()
        if cur and size + b > limit:
            groups.append(cur)
            cur, size = {}, 0
        cur[n] = t
        size += b
        total += b
    if cur or not groups:
        groups.append(cur)
    if len(groups) == 1:
        return {weights_name: groups[0]}, None
    stem, ext = os.path.splitext(weights_name)
    shards, weight_map = {}, {}
    for i, g in enumerate(groups):
        fname = f"{stem}-{i + 1:05d}-of-{len(groups):05d}{ext}"
        shards[fname] = g
        weight_map.update({n: fname for n in g})
    return shards, {"metadata": {"total_size": total}, "weight_map": weight_map}


def _size_to_int(text) -> int:
    s = str(text).strip().upper()
    for unit, mul in (("GIB", 1 << 30), ("MIB", 1 << 20), ("KIB", 1 << 10), ("GB", 10 ** 9), ("MB", 10 ** 6), ("KB", 10 ** 3)):
        if s.endswith(unit):
            return int(float(s[:-len(unit)]) * mul)
    return int(s)


def save_pretrained_dir(model: torch.nn.Module, directory: str, config_dict: Optional[dict] = None,
                        max_shard_bytes: int = 5 << 30, hf_names: bool = False, family: str = "llama"):
    """HF-style directory: ``config.json`` + (sharded) ``model-0000x-of-0000y.safetensors`` + index."""
    os.makedirs(directory, exist_ok=True)
    sd = {n: t.contiguous().cpu() for n, t in model_state(model).items()}
    if hf_names:
        sd = name_maps.framework_to_hf(sd, model.config, family)
    shards, index = shard_checkpoint(sd, max_shard_bytes, "model.safetensors")
    for fname, part in shards.items():
        save_file(part, os.path.join(directory, fname), metadata={"format": "pt"})
    if index is not None:
        with open(os.path.join(directory, "model.safetensors.index.json"), "w") as f:
            json.dump(index, f, indent=1)
    if config_dict is not None:
        with open(os.path.join(directory, "config.json"), "w") as f:
            json.dump(config_dict, f, indent=1, default=str)
