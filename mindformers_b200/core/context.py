"""Process-wide runtime context: device, seed, determinism, distributed initialisation.

Mirrors the API of the reference's ``core/context/build_context.py`` (``build_context`` :431, ``init_context``,
``set_context``, ``get_context`` :396-566, ``Context`` singleton :46-91) and ``core/context/parallel.py``
(``init_communication`` :83-100). Ascend/MindSpore keys are accepted and mapped where a CUDA meaning exists:
``device_id`` → CUDA device, ``max_device_memory`` → per-process memory fraction, ``train_precision_sync`` /
``infer_precision_sync`` → deterministic algorithms + ``NCCL_ALGO=Ring``, ``CPU_AFFINITY`` → ``sched_setaffinity``.
"""
from __future__ import annotations

import os
import random
from typing import Optional

import numpy as np
import torch
import torch.distributed as dist

from ..parallel import parallel_state as ps
from ..tools.logger import logger
from ..tools.register import set_use_legacy

_CONTEXT = None


def _parse_mem(value) -> Optional[float]:
    if value is None:
        return None
    s = str(value).strip().upper()
    if s.endswith("GB"):
        return float(s[:-2]) * (1 << 30)
    if s.endswith("MB"):
        return float(s[:-2]) * (1 << 20)
    return float(s)


def resolve_3d_tensor_parallel(par, model_cfg) -> Optional[dict]:
    """``use_3d_tensor_parallel`` with ``tp_x``, ``tp_y``, ``tp_z`` (reference ``modules/flash_attention.py:148-164,
    352-353`` and ``modules/layers.py:1549-1551``): the model-parallel devices form a ``z x x x y`` grid on which an
    activation ``[batch, heads, sequence, head_dim]`` is laid out with the heads over ``y`` and the sequence over
    ``(cp, z, x)``. The same layout here is tensor parallelism of size ``tp_y`` (heads, and the rows / columns of the
    linear layers) with context parallelism of size ``cp * tp_z * tp_x`` (the sequence); both settings are rewritten
    in place, so every later reader of ``parallel_config`` (group construction, model configuration) sees the
    two-level layout. Returns the resolved sizes, or None when the model does not ask for it."""
    if model_cfg is None or not hasattr(model_cfg, "get") or not model_cfg.get("use_3d_tensor_parallel"):
        return None
    x, y, z = (int(model_cfg.get(k, 1) or 1) for k in ("tp_x", "tp_y", "tp_z"))
    mp = int(par.get("model_parallel", 1) or 1)
    done = par.get("_tensor_parallel_3d")
    if done:
        return dict(done)
    if min(x, y, z) < 1 or x * y * z != mp:
        raise ValueError(f"use_3d_tensor_parallel: tp_x * tp_y * tp_z = {x} * {y} * {z} must equal model_parallel = {mp}")
    if model_cfg.get("use_seq_parallel") or par.get("use_seq_parallel"):
        raise ValueError("use_3d_tensor_parallel cannot be combined with use_seq_parallel (the reference rejects it too)")
    cp = int(par.get("context_parallel", 1) or 1)
    out = {"tp_x": x, "tp_y": y, "tp_z": z, "model_parallel": y, "context_parallel": cp * x * z}
    par["model_parallel"], par["context_parallel"] = out["model_parallel"], out["context_parallel"]
    par["_tensor_parallel_3d"] = dict(out)
    logger.info("3-D tensor parallelism %d x %d x %d: heads over %d devices, sequence over %d", x, y, z, y, cp * x * z)
    return out


class Context:
    """Singleton holding the effective settings."""

    def __init__(self, config=None):
        cfg = config or {}
        self.config = cfg
        ctx = dict(cfg.get("context") or {})
        raw_par = cfg.get("parallel_config") if hasattr(cfg, "get") else None
        model_cfg = (cfg.get("model") or {}).get("model_config") if hasattr(cfg, "get") and cfg.get("model") else None
        if raw_par is not None and hasattr(raw_par, "get"):
            # rewrites model_parallel / context_parallel in the configuration itself: the model builder reads them too
            self.tensor_parallel_3d = resolve_3d_tensor_parallel(raw_par, model_cfg)
        else:
            self.tensor_parallel_3d = None
        par = dict(raw_par or {})
        self.use_parallel = bool(cfg.get("use_parallel", False))
        self.run_mode = cfg.get("run_mode")
        self.seed = cfg.get("seed", 1)
        self.device_target = str(ctx.get("device_target", "CUDA")).upper()
        self.local_rank = int(os.environ.get("LOCAL_RANK", ctx.get("device_id", 0) or 0))
        self.settings = dict(ctx)
        self.parallel_settings = par
        set_use_legacy(cfg.get("use_legacy", True))
        if self.run_mode:
            os.environ["RUN_MODE"] = str(self.run_mode)
        self._set_device(ctx)
        self._set_determinism(cfg)
        self._set_affinity()
        self.parallel_speed_up = self._load_parallel_speed_up(cfg, ctx)
        self.set_seed(self.seed)
        self.rank, self.world_size = 0, 1
        if self.use_parallel:
            self.init_communication(par)

    # ----------------------------------------------------------------------------------------------
    # keys of a ``parallel_speed_up.json`` that have a counterpart here: overlap of a GEMM with its collective is what
    # the fused kernels do, so these switch them on (model_config keys) unless the YAML already says otherwise
    _SPEED_UP_MAP = {"matmul_grad_comm_overlap": "fused_tp_comm", "enable_grad_comm_opt": "fused_tp_comm",
                     "enable_opt_shard_comm_opt": "fused_tp_comm", "compute_communicate_fusion_level": "fused_tp_comm",
                     "enable_concat_eliminate_opt": None, "enable_begin_end_inline_opt": None,
                     "dataset_broadcast_opt_level": None, "recompute_comm_overlap": None}

    def _load_parallel_speed_up(self, cfg, ctx) -> dict:
        """``context.ascend_config.parallel_speed_up_json_path`` (reference ``configs/qwen3/parallel_speed_up.json``,
        ``research/qwen2_5/parallel_speed_up_72B_32K.json``): graph-compiler knobs of the reference's backend. Those
        that mean "overlap this GEMM with its collective" select the fused communication kernels; the others have
        nothing to steer here and are listed as ignored."""
        path = (ctx.get("ascend_config") or {}).get("parallel_speed_up_json_path") or ctx.get("parallel_speed_up_json_path")
        out = {"path": path, "applied": {}, "ignored": []}
        if not path:
            return out
        if not os.path.exists(path):
            logger.warning("parallel_speed_up_json_path %s does not exist; ignored", path)
            return out
        import json
        with open(path) as f:
            knobs = json.load(f)
        model_cfg = ((cfg.get("model") or {}).get("model_config")) if hasattr(cfg, "get") else None
        for key, value in knobs.items():
            target = self._SPEED_UP_MAP.get(key)
            if target and value:
                out["applied"][key] = target
                if model_cfg is not None and model_cfg.get(target) is None:
                    model_cfg[target] = True
            else:
                out["ignored"].append(key)
        logger.info("parallel_speed_up: applied %s, ignored %s", out["applied"], out["ignored"])
        return out

    def _set_device(self, ctx):
        if torch.cuda.is_available() and self.device_target not in ("CPU",):
            torch.cuda.set_device(self.local_rank % torch.cuda.device_count())
            self.device = torch.device("cuda", torch.cuda.current_device())
            limit = _parse_mem(ctx.get("max_device_memory"))
            if limit:
                total = torch.cuda.get_device_properties(self.device).total_memory
                torch.cuda.set_per_process_memory_fraction(min(1.0, limit / total), self.device)
        else:
            self.device = torch.device("cpu")

    def _set_determinism(self, cfg):
        train_sync, infer_sync = cfg.get("train_precision_sync"), cfg.get("infer_precision_sync")
        on = bool(train_sync) or bool(infer_sync)
        if train_sync is not None or infer_sync is not None:
            torch.use_deterministic_algorithms(on, warn_only=True)
            torch.backends.cudnn.deterministic = on
            torch.backends.cudnn.benchmark = not on
            if on:
                os.environ.setdefault("NCCL_ALGO", "Ring")
                os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
        self.deterministic = on

    def _set_affinity(self):
        if os.environ.get("CPU_AFFINITY", "").lower() in ("1", "true") and hasattr(os, "sched_setaffinity"):
            n = os.cpu_count() or 1
            per = max(1, n // max(1, torch.cuda.device_count() or 1))
            cores = set(range(self.local_rank * per, min(n, (self.local_rank + 1) * per)))
            if cores:
                try:
                    os.sched_setaffinity(0, cores)
                except OSError as e:  # pragma: no cover - depends on the container
                    logger.warning("cannot set CPU affinity: %s", e)

    @staticmethod
    def set_seed(seed: int):
        random.seed(seed)
        np.random.seed(seed % (2 ** 32))
        torch.manual_seed(seed)

    def choose_pipeline_stages(self, par: dict, auto: bool = False) -> int:
        """``parallel_config.pipeline_stage``, or with ``parallel.auto_pipeline`` the reference's rule
        (``core/context/parallel.py:46-64``): ``min(max(stages given, number of servers), micro_batch_num)``, so that a
        job spread over several nodes pipelines across them (the slow links carry activations only) but never uses more
        stages than there are micro-batches to fill them. The result must divide the device count left after tensor and
        context parallelism; the largest such value not above the rule's is taken."""
        given = int(par.get("pipeline_stage", 1) or 1)
        if not auto:
            return given
        local = int(os.environ.get("LOCAL_WORLD_SIZE", 0) or 0) or max(torch.cuda.device_count(), 1)
        servers = max(1, self.world_size // max(local, 1))
        micro = int(par.get("micro_batch_num", 1) or 1)
        want = min(max(given, servers), micro)
        rest = self.world_size // (int(par.get("model_parallel", 1) or 1) * int(par.get("context_parallel", 1) or 1))
        while want > 1 and rest % want:
            want -= 1
        if par.get("data_parallel") and want != given:
            par["data_parallel"] = rest // want
        logger.info("automatic pipeline stages: %d (given %d, servers %d, micro batches %d)", want, given, servers, micro)
        return max(want, 1)

    def init_communication(self, par: dict):
        """Join the job (``torchrun`` environment) and build the model-parallel groups."""
        if "RANK" not in os.environ:
            logger.warning("use_parallel is set but no launcher environment was found; running single process")
            return
        if not dist.is_initialized():
            backend = "nccl" if self.device.type == "cuda" else "gloo"
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            kwargs = {"device_id": self.device} if backend == "nccl" else {}
            dist.init_process_group(backend, **kwargs)
        self.rank, self.world_size = dist.get_rank(), dist.get_world_size()
        tp = int(par.get("model_parallel", 1) or 1)
        pp = self.choose_pipeline_stages(par, ((self.config or {}).get("parallel") or {}).get("auto_pipeline"))
        if pp != int(par.get("pipeline_stage", 1) or 1):
            par["pipeline_stage"] = pp
        cp = int(par.get("context_parallel", 1) or 1)
        ep = int(par.get("expert_parallel", 1) or 1)
        dp = par.get("data_parallel")
        expect = tp * pp * cp * int(dp or self.world_size // (tp * pp * cp))
        if expect != self.world_size:
            raise ValueError(f"data_parallel*model_parallel*context_parallel*pipeline_stage = {expect} does not "
                             f"match the number of devices {self.world_size}")
        ps.initialize_model_parallel(tensor_model_parallel_size=tp, pipeline_model_parallel_size=pp,
                                     context_parallel_size=cp, expert_model_parallel_size=ep,
                                     expert_tensor_parallel_size=par.get("expert_model_parallel"),
                                     virtual_pipeline_model_parallel_size=(par.get("pp_interleave_num") or None)
                                     if (par.get("pp_interleave_num") or 1) > 1 else None)


def build_context(config=None) -> Context:
    """Create (or replace) the process context from a full configuration mapping."""
    global _CONTEXT
    _CONTEXT = Context(config)
    return _CONTEXT


def init_context(use_parallel: bool = False, context_config: Optional[dict] = None,
                 parallel_config: Optional[dict] = None):
    """Older two-argument form; returns ``(local_rank, world_size)``."""
    ctx = build_context({"use_parallel": use_parallel, "context": context_config or {},
                         "parallel_config": parallel_config or {}})
    return ctx.local_rank, ctx.world_size


def get_context(key: Optional[str] = None):
    if _CONTEXT is None:
        raise RuntimeError("build_context() has not been called")
    if key is None:
        return _CONTEXT
    if hasattr(_CONTEXT, key):
        return getattr(_CONTEXT, key)
    return _CONTEXT.settings.get(key)


def set_context(**kwargs):
    if _CONTEXT is None:
        raise RuntimeError("build_context() has not been called")
    for k, v in kwargs.items():
        if k == "seed":
            _CONTEXT.set_seed(v)
            _CONTEXT.seed = v
        elif k in ("train_precision_sync", "infer_precision_sync"):
            _CONTEXT._set_determinism({k: v})
        else:
            _CONTEXT.settings[k] = v


def is_context_built() -> bool:
    return _CONTEXT is not None


from .._submodules import alias_children as _alias_children  # noqa: E402

_alias_children(__name__, ['build_context', 'parallel', 'validators'])
