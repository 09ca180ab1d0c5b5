"""Training callbacks: monitors, checkpointing, profiling, anomaly handling.

What each class answers to in the reference (``mindformers/core/callback/callback.py``):
``MFLossMonitor`` :167-537 (per-step loss / time / lr / norm / throughput line and TensorBoard scalars),
``TrainingStateMonitor`` :540-1055 (local norms, NaN and spike checks, skip-data bookkeeping),
``SummaryMonitor`` :1057, ``CheckpointMonitor`` :1119-1645 (three outputs, rotation, ``meta.json``, health
flag), ``ProfileMonitor`` :1649-1916, ``EvalCallBack`` :1919, ``ColdHotExpertMonitor`` :1979,
``StressDetectCallBack`` :2175, ``TopkBiasBalanceCallback`` :2241-2337, ``MoEDropRateCallback`` :2339,
``SDCMonitor`` :2703 and the fault-tolerance callback wired in ``trainer/base_trainer.py:1095-1125``.

The protocol is plain Python: the trainer owns a ``RunContext`` and calls ``on_train_begin``,
``on_step_begin``, ``on_step_end``, ``on_epoch_end``, ``on_train_end`` on every callback. Step time is
taken from CUDA events recorded by the trainer on the compute stream, so the monitor adds no device
synchronisation of its own beyond the loss read that the user asked for.
"""
from __future__ import annotations

import json
import math
import os
import re
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional

import torch

from ..tools.logger import get_logger
from ..tools.register.register import MindFormerModuleType, MindFormerRegister
from ..tools.utils import get_output_root_path, get_real_group_size, get_real_rank

logger = get_logger()


@dataclass
class RunContext:
    """Mutable view of the run that callbacks read (and, for ``request_stop``, write)."""
    engine: Any = None
    config: Any = None
    epoch: int = 0
    epochs: int = 1
    step_in_epoch: int = 0
    steps_per_epoch: int = 0
    global_step: int = 0
    total_steps: int = 0
    global_batch_size: int = 1
    seq_length: int = 0
    loss: Optional[float] = None
    lr: Optional[float] = None
    global_norm: Optional[float] = None
    skipped: bool = False
    loss_scale: float = 1.0
    step_ms: float = 0.0
    extras: Dict[str, Any] = field(default_factory=dict)
    request_stop: bool = False
    stop_reason: str = ""


class Callback:
    """Hooks that the training loop calls: ``on_train_begin/end``, ``on_epoch_begin/end``, ``on_step_begin/end``,
    each with the ``RunContext``."""

    def on_train_begin(self, ctx: RunContext): ...
    def on_step_begin(self, ctx: RunContext): ...
    def on_step_end(self, ctx: RunContext): ...
    def on_epoch_end(self, ctx: RunContext): ...
    def on_train_end(self, ctx: RunContext): ...
    def on_exception(self, ctx: RunContext, exc: BaseException): ...


def _reg(cls):
    MindFormerRegister.register_cls(cls, MindFormerModuleType.CALLBACK)
    return cls


def model_flops_per_token(cfg, seq_length: int) -> float:
    """Forward+backward matmul FLOPs per token of a decoder-only model (analytic; the reference asks the
    graph compiler, ``callback.py:385-423``). Causal attention counts half of the full score matrix."""
    h, L = cfg.hidden_size, cfg.num_layers
    hd = getattr(cfg, "kv_channels", None) or h // cfg.num_attention_heads
    nq, nkv = cfg.num_attention_heads, (cfg.num_query_groups or cfg.num_attention_heads)
    attn_proj = 2 * h * (nq * hd + 2 * nkv * hd) + 2 * nq * hd * h
    attn_core = 2 * 2 * seq_length * nq * hd / 2
    ffn = cfg.ffn_hidden_size
    if getattr(cfg, "num_moe_experts", None):
        moe_ffn = (cfg.moe_ffn_hidden_size or ffn)
        mlp = 2 * 3 * h * moe_ffn * cfg.moe_router_topk + 2 * h * cfg.num_moe_experts
        if cfg.moe_shared_expert_intermediate_size:
            mlp += 2 * 3 * h * cfg.moe_shared_expert_intermediate_size
    else:
        mlp = 2 * 3 * h * ffn if cfg.gated_linear_unit else 2 * 2 * h * ffn
    head = 2 * h * cfg.vocab_size
    return 3.0 * (L * (attn_proj + attn_core + mlp) + head)


@_reg
class MFLossMonitor(Callback):
    """One log line per ``per_print_times`` steps plus optional TensorBoard scalars."""

    def __init__(self, learning_rate=None, per_print_times: int = 1, micro_batch_num: int = 1,
                 micro_batch_interleave_num: int = 1, origin_epochs: Optional[int] = None, dataset_size: Optional[int] = None,
                 initial_epoch: int = 0, initial_step: int = 0, global_batch_size: int = 0, gradient_accumulation_steps: int = 1,
                 check_for_nan_in_loss_and_grad: bool = False, calculate_per_token_loss: bool = False,
                 print_separate_loss: bool = False, tensorboard_writer=None, **kwargs):
        self.per_print_times = max(1, per_print_times)
        self.check_nan = check_for_nan_in_loss_and_grad
        self.tb = tensorboard_writer
        self.history: List[Dict[str, float]] = []
        self._t0 = None
        self.global_batch_size = global_batch_size

    def on_train_begin(self, ctx):
        self._t0 = time.time()

    def on_step_end(self, ctx):
        gbs = self.global_batch_size or ctx.global_batch_size
        world = get_real_group_size()
        step_s = max(ctx.step_ms, 1e-6) / 1e3
        samples_per_s_per_dev = gbs / world / step_s          # callback.py:313
        tokens_per_s = gbs * ctx.seq_length / step_s
        rec = dict(step=ctx.global_step, loss=ctx.loss, lr=ctx.lr, global_norm=ctx.global_norm, step_ms=ctx.step_ms,
                   samples_per_s_per_device=samples_per_s_per_dev, tokens_per_s=tokens_per_s, skipped=ctx.skipped)
        tcfg = getattr(getattr(ctx.engine, "model", None), "config", None)
        if tcfg is not None and ctx.seq_length:
            try:
                rec["model_tflops_per_device"] = model_flops_per_token(tcfg, ctx.seq_length) * tokens_per_s / world / 1e12
            except Exception:  # pragma: no cover - config without the needed fields
                pass
        self.history.append(rec)
        if self.check_nan and ctx.loss is not None and not math.isfinite(ctx.loss):
            raise ValueError(f"loss is {ctx.loss} at step {ctx.global_step}")
        if ctx.global_step % self.per_print_times == 0 and get_real_rank() == 0:
            done = ctx.global_step / max(ctx.total_steps, 1)
            eta = (ctx.total_steps - ctx.global_step) * step_s
            logger.info("{ Epoch:[%3d/%3d], step:[%5d/%5d], loss: %.6f, per_step_time: %dms, lr: %s, overflow cond: %s, "
                        "loss_scale: %s, global_norm: %s, train_throughput_per_device: %.3fT, samples/s/p: %.3f, "
                        "tokens/s: %.1f, %.1f%% , eta %ds }", ctx.epoch + 1, ctx.epochs, ctx.step_in_epoch,
                        ctx.steps_per_epoch, ctx.loss if ctx.loss is not None else float("nan"), int(ctx.step_ms),
                        f"{ctx.lr:.6e}" if ctx.lr is not None else "-", ctx.skipped, ctx.loss_scale,
                        f"{ctx.global_norm:.4f}" if ctx.global_norm is not None else "-",
                        rec.get("model_tflops_per_device", 0.0), samples_per_s_per_dev, tokens_per_s, 100 * done, int(eta))
        if self.tb is not None:
            seen = ctx.global_step * gbs
            for tag, val in (("learning-rate", ctx.lr), ("batch-size", gbs), ("loss", ctx.loss), ("grad-norm", ctx.global_norm),
                             ("iteration-time", step_s), ("throughput", rec.get("model_tflops_per_device")),
                             ("B-samples-per-day", samples_per_s_per_dev * world * 86400 / 1e9)):
                if val is not None:
                    self.tb.add_scalar(tag, val, ctx.global_step)
                    self.tb.add_scalar(f"{tag} vs samples", val, seen)


@_reg
class SummaryMonitor(Callback):
    """Scalar summaries to TensorBoard every ``collect_freq`` steps."""

    def __init__(self, summary_dir: Optional[str] = None, collect_freq: int = 10, **kwargs):
        from ..utils.tensorboard import get_tensorboard_writer
        self.writer = get_tensorboard_writer(summary_dir or os.path.join(get_output_root_path(), "summary"))
        self.freq = max(1, collect_freq)

    def on_step_end(self, ctx):
        if self.writer is not None and ctx.global_step % self.freq == 0 and ctx.loss is not None:
            self.writer.add_scalar("summary/loss", ctx.loss, ctx.global_step)


@_reg
class TrainingStateMonitor(Callback):
    """Norm / loss anomaly detection and optional per-parameter statistics.

    * NaN / Inf loss or global norm → ``RuntimeError`` (reference :1048).
    * global-norm spike (``global_norm_spike_threshold``): the step number is appended to
      ``global_norm_spike_record.json`` and, unless ``check_for_global_norm`` is off, a
      ``RuntimeError("TREError ...")`` is raised so that a supervisor can roll back (:770-789).
    * skip-data: consecutive skipped steps are counted and the run aborts after
      ``global_norm_spike_count_threshold`` of them (:791-811).
    * ``local_norm`` / ``weight_state_format`` / ``optimizer_state_format``: per-parameter L2 norms
      (regex ``target``) logged or written to TensorBoard.
    """

    def __init__(self, origin_epochs: int = 1, config: Optional[dict] = None, step_interval: int = 1, dataset_size: int = 0,
                 initial_epoch: int = 0, initial_step: int = 0, global_batch_size: int = 0, check_for_nan_in_loss_and_grad: bool = True,
                 use_skip_data_by_global_norm: bool = False, tensorboard_writer=None, **kwargs):
        cfg = dict(config or {})
        cfg.update(kwargs)
        self.step_interval = max(1, cfg.get("step_interval", step_interval))
        self.target = [re.compile(p) for p in (cfg.get("target") or [".*"])]
        self.local_norm_format = cfg.get("local_norm_format")
        self.weight_state_format = cfg.get("weight_state_format")
        self.optimizer_state_format = cfg.get("optimizer_state_format")
        self.local_loss_format = cfg.get("local_loss_format")
        self.throughput_baseline = cfg.get("throughput_baseline")
        self.spike_threshold = float(cfg.get("global_norm_spike_threshold", 0) or 0)
        self.spike_count_threshold = int(cfg.get("global_norm_spike_count_threshold", 10))
        self.check_for_global_norm = bool(cfg.get("check_for_global_norm", False))
        self.record_path = cfg.get("global_norm_record_path") or os.path.join(get_output_root_path(), "global_norm_spike_record.json")
        self.check_nan = check_for_nan_in_loss_and_grad
        self.use_skip = use_skip_data_by_global_norm
        self.tb = tensorboard_writer
        self.consecutive_skips = 0
        self.stats: List[Dict[str, Any]] = []

    def _match(self, name):
        return any(p.search(name) for p in self.target)

    def _emit(self, fmt, tag, value, step):
        fmts = fmt if isinstance(fmt, (list, tuple)) else [fmt]
        if "log" in fmts:
            logger.info("%s: %.6f", tag, value)
        if "tensorboard" in fmts and self.tb is not None:
            self.tb.add_scalar(tag, value, step)

    def on_step_end(self, ctx):
        for name, val in (("loss", ctx.loss), ("global_norm", ctx.global_norm)):
            if self.check_nan and val is not None and not math.isfinite(val):
                raise RuntimeError(f"{name} is {val} at step {ctx.global_step}")
        if ctx.skipped:
            self.consecutive_skips += 1
            if self.use_skip and self.consecutive_skips >= self.spike_count_threshold:
                raise RuntimeError(f"{self.consecutive_skips} consecutive steps skipped by the global-norm threshold; "
                                   f"stopping at step {ctx.global_step}")
        else:
            self.consecutive_skips = 0
        if self.spike_threshold and ctx.global_norm is not None and ctx.global_norm >= self.spike_threshold:
            rec = {}
            if os.path.exists(self.record_path):
                with open(self.record_path) as f:
                    rec = json.load(f)
            rec.setdefault(str(ctx.global_step), []).append(ctx.global_norm)
            os.makedirs(os.path.dirname(self.record_path) or ".", exist_ok=True)
            tmp = self.record_path + ".tmp"
            with open(tmp, "w") as f:
                json.dump(rec, f)
            os.replace(tmp, self.record_path)
            if self.check_for_global_norm:
                raise RuntimeError(f"TREError occurred: global norm {ctx.global_norm:.4f} >= {self.spike_threshold} "
                                   f"at step {ctx.global_step}")
        if ctx.global_step % self.step_interval:
            return
        model = getattr(ctx.engine, "model", None)
        snap: Dict[str, Any] = {"step": ctx.global_step}
        if model is not None and self.weight_state_format:
            for n, p in model.named_parameters():
                if self._match(n):
                    v = float(p.detach().float().norm())
                    snap[f"weight_norm/{n}"] = v
                    self._emit(self.weight_state_format, f"weight_norm/{n}", v, ctx.global_step)
        if model is not None and self.local_norm_format:
            for n, g in ctx.extras.get("local_norms", {}).items():
                if self._match(n):
                    snap[f"local_norm/{n}"] = g
                    self._emit(self.local_norm_format, f"local_norm/{n}", g, ctx.global_step)
        opt = getattr(ctx.engine, "optimizer", None)
        if opt is not None and self.optimizer_state_format and hasattr(opt, "state_norms"):
            for n, v in opt.state_norms().items():
                snap[f"optimizer/{n}"] = v
                self._emit(self.optimizer_state_format, f"optimizer/{n}", v, ctx.global_step)
        if self.throughput_baseline and ctx.step_ms:
            tput = ctx.global_batch_size / (ctx.step_ms / 1e3) / get_real_group_size()
            snap["throughput_linearity"] = tput / self.throughput_baseline
        self.stats.append(snap)


@_reg
class CheckpointMonitor(Callback):
    """Periodic checkpoints under ``<output>/checkpoint/rank_N/{prefix}_rank_N-{epoch}_{step}.safetensors``.

    Saves by step interval (``save_checkpoint_steps``) or wall-clock interval (``save_checkpoint_seconds``), keeps
    ``keep_checkpoint_max`` files per rank, optionally a weights-only copy (``save_network_params`` →
    ``checkpoint_network/``) and a trainable-only copy (``save_trainable_params`` → ``checkpoint_trainable/``),
    records ``meta.json`` atomically and, with ``use_checkpoint_health_monitor``, flags a checkpoint whose
    embedding norm is below ``embedding_local_norm_threshold`` as unhealthy so that resume skips it.
    ``exception_save`` writes one last checkpoint when the training loop raises.
    """

    def __init__(self, prefix: str = "CKP", directory: Optional[str] = None, config=None, save_checkpoint_steps: int = 1,
                 save_checkpoint_seconds: int = 0, keep_checkpoint_max: int = 5, keep_checkpoint_per_n_minutes: int = 0,
                 integrated_save: bool = False, save_network_params: bool = False, save_trainable_params: bool = False,
                 async_save: bool = False, saved_network=None, append_info=None, checkpoint_format: str = "safetensors",
                 remove_redundancy: bool = False, exception_save: bool = False, global_batch_size: Optional[int] = None,
                 use_checkpoint_health_monitor: bool = False, health_ckpts_record_dir: Optional[str] = None,
                 embedding_local_norm_threshold: float = 1.0, use_legacy_format: bool = False, **kwargs):
        if checkpoint_format not in ("safetensors",):
            raise ValueError(f"checkpoint_format {checkpoint_format!r}: only 'safetensors' is written by this framework")
        self.prefix = prefix
        self.directory = directory
        self.every_steps = int(save_checkpoint_steps or 0)
        self.every_seconds = int(save_checkpoint_seconds or 0)
        self.keep_max = keep_checkpoint_max
        self.save_network = save_network_params
        self.save_trainable = save_trainable_params
        self.async_save = async_save
        self.remove_redundancy = remove_redundancy
        self.exception_save = exception_save
        self.global_batch_size = global_batch_size
        self.health = use_checkpoint_health_monitor
        self.health_threshold = embedding_local_norm_threshold
        self._last_time = time.time()
        self._last_saved_step = -1
        self._pending = None
        self.saved: List[str] = []

    def _dir(self):
        return self.directory or os.path.join(get_output_root_path(), "checkpoint")

    def _wait_async(self):
        if self._pending is not None:
            self._pending.join()
            self._pending = None

    def save(self, ctx: RunContext, tag_exception: bool = False) -> Optional[str]:
        from ..checkpoint.io import save_checkpoint
        from ..checkpoint.resume import mark_unhealthy
        engine = ctx.engine
        if engine is None or ctx.global_step == self._last_saved_step:
            return None
        self._wait_async()
        extra = {"global_batch_size": self.global_batch_size or ctx.global_batch_size, "loss_scale": float(ctx.loss_scale)}
        kw = dict(optimizer=getattr(engine, "optimizer", None), prefix=self.prefix, epoch=ctx.epoch + 1,
                  step=ctx.step_in_epoch, extra=extra, keep_max=self.keep_max, save_network_only_copy=self.save_network,
                  remove_redundancy=self.remove_redundancy)
        t0 = time.time()
        if self.async_save and not tag_exception:
            # the state is copied to pinned host memory on the training stream before this returns; the thread only
            # writes those copies, so steps that run meanwhile cannot leak into the file
            import threading
            from ..checkpoint.io import snapshot_checkpoint, write_checkpoint
            from ..checkpoint.sharding import save_strategy
            from ..tools.utils import get_real_rank
            d, rank = self._dir(), get_real_rank()
            root = os.path.dirname(d.rstrip("/")) or "."
            snap = snapshot_checkpoint(engine.model, optimizer=kw["optimizer"], epoch=kw["epoch"], step=kw["step"],
                                       extra=extra, remove_redundancy=self.remove_redundancy)
            save_strategy(engine.model, os.path.join(root, "strategy", f"ckpt_strategy_rank_{rank}.json"))
            wkw = dict(rank=rank, prefix=self.prefix, epoch=kw["epoch"], step=kw["step"], keep_max=self.keep_max,
                       remove_redundancy=self.remove_redundancy,
                       network_only_dir=os.path.join(root, "checkpoint_network") if self.save_network else None)
            th = threading.Thread(target=lambda: self.saved.append(write_checkpoint(snap, d, **wkw)), daemon=True)
            th.start()
            self._pending = th
            path = None
        else:
            path = save_checkpoint(engine.model, self._dir(), **kw)
            self.saved.append(path)
        if self.save_trainable:
            tdir = os.path.join(os.path.dirname(self._dir().rstrip("/")) or ".", "checkpoint_trainable")
            save_checkpoint(engine.model, tdir, prefix=self.prefix, epoch=ctx.epoch + 1, step=ctx.step_in_epoch,
                            keep_max=self.keep_max, trainable_only=True, write_strategy=False)
        if self.health:
            emb = [p for n, p in engine.model.named_parameters() if "word_embeddings" in n]
            if emb and float(emb[0].detach().float().norm()) < self.health_threshold:
                mark_unhealthy(self._dir(), ctx.epoch + 1, ctx.step_in_epoch, "embedding norm below threshold")
        self._last_saved_step = ctx.global_step
        self._last_time = time.time()
        logger.info("checkpoint at epoch %d step %d saved in %.2fs%s", ctx.epoch + 1, ctx.step_in_epoch,
                    time.time() - t0, " (exception save)" if tag_exception else "")
        return path

    def on_step_end(self, ctx):
        due = self.every_steps and ctx.global_step % self.every_steps == 0
        if self.every_seconds and time.time() - self._last_time >= self.every_seconds:
            due = True
        if due:
            self.save(ctx)

    def on_train_end(self, ctx):
        self.save(ctx)
        self._wait_async()

    def on_exception(self, ctx, exc):
        if self.exception_save:
            try:
                self.save(ctx, tag_exception=True)
            except Exception as e:  # pragma: no cover - best effort
                logger.error("exception save failed: %s", e)


@_reg
class ProfileMonitor(Callback):
    """``torch.profiler`` window ``[start_step, stop_step)`` with NVTX step ranges.

    Keys follow the reference (:1649-1916): ``start_step, stop_step, output_path, profile_rank_ids,
    profile_pipeline, profile_communication, profile_memory, with_stack, profiler_level``; traces land in
    ``<output>/profile/rank_N`` in TensorBoard/Chrome-trace format together with the parallel layout as metadata.
    """

    def __init__(self, start_step: int = 1, stop_step: int = 10, output_path: Optional[str] = None, start_profile: bool = True,
                 profile_rank_ids: Optional[List[int]] = None, profile_pipeline: bool = False, profile_communication: bool = False,
                 profile_memory: bool = False, config=None, profiler_level: int = 0, with_stack: bool = False,
                 data_simplification: bool = True, mstx: bool = False, **kwargs):
        self.start_step, self.stop_step = start_step, stop_step
        rank = get_real_rank()
        self.dir = os.path.join(output_path or os.path.join(get_output_root_path(), "profile"), f"rank_{rank}")
        ranks = profile_rank_ids
        if ranks is None and profile_pipeline:
            from ..tools.utils import get_pipeline_rank_ids
            ranks = get_pipeline_rank_ids()
        self.enabled = ranks is None or rank in ranks
        self.profile_memory, self.with_stack, self.nvtx = profile_memory, with_stack, mstx
        self.prof = None
        self.meta = dict(config or {})

    def on_step_begin(self, ctx):
        if not self.enabled:
            return
        if self.nvtx and torch.cuda.is_available():
            torch.cuda.nvtx.range_push(f"step {ctx.global_step + 1}")
        if ctx.global_step + 1 == self.start_step and self.prof is None:
            acts = [torch.profiler.ProfilerActivity.CPU]
            if torch.cuda.is_available():
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            os.makedirs(self.dir, exist_ok=True)
            self.prof = torch.profiler.profile(activities=acts, profile_memory=self.profile_memory, with_stack=self.with_stack,
                                               on_trace_ready=torch.profiler.tensorboard_trace_handler(self.dir))
            self.prof.__enter__()

    def on_step_end(self, ctx):
        if not self.enabled:
            return
        if self.nvtx and torch.cuda.is_available():
            torch.cuda.nvtx.range_pop()
        if self.prof is not None:
            self.prof.step()
            if ctx.global_step >= self.stop_step:
                self._finish()

    def _finish(self):
        if self.prof is not None:
            self.prof.__exit__(None, None, None)
            self.prof = None
            with open(os.path.join(self.dir, "parallel_config.json"), "w") as f:
                json.dump(self.meta, f, default=str)

    def on_train_end(self, ctx):
        self._finish()


@_reg
class EvalCallBack(Callback):
    """Runs ``eval_func`` every ``step_interval`` steps and/or ``epoch_interval`` epochs."""

    def __init__(self, eval_func: Callable[[], Any], step_interval: int = 100, epoch_interval: int = -1, **kwargs):
        self.fn, self.step_interval, self.epoch_interval = eval_func, step_interval, epoch_interval
        self.results: List[Any] = []

    def on_step_end(self, ctx):
        if self.step_interval > 0 and ctx.global_step % self.step_interval == 0:
            self.results.append(self.fn())

    def on_epoch_end(self, ctx):
        if self.epoch_interval > 0 and (ctx.epoch + 1) % self.epoch_interval == 0:
            self.results.append(self.fn())


@_reg
class TopkBiasBalanceCallback(Callback):
    """Aux-loss-free balancing: after each step nudges every router's ``expert_bias`` against its load by
    ``balance_via_topk_bias``' update rate and logs the per-layer load (:2241-2337)."""

    def __init__(self, balance_via_topk_bias: bool = False, topk_bias_update_rate: float = 0.0, expert_num: int = 0,
                 micro_batch_num: int = 1, gradient_accumulation_steps: int = 1, tensorboard_writer=None,
                 dump_dir: Optional[str] = None, **kwargs):
        self.enabled, self.tb = balance_via_topk_bias, tensorboard_writer
        self.loads: List[Dict[str, List[float]]] = []
        # ``dump_dir``: one ``layer-<L>-step<N>.npy`` per MoE layer and step, the input of
        # ``tools/moe_token_distribution_tools.py``
        self.dump_dir = dump_dir

    def on_step_end(self, ctx):
        model = getattr(ctx.engine, "model", None)
        if model is None:
            return
        snap = {}
        for n, m in model.named_modules():
            load = getattr(m, "expert_load", None)
            if load is not None:
                snap[n] = load.detach().float().cpu().tolist()
                if self.tb is not None:
                    for e, v in enumerate(snap[n]):
                        self.tb.add_scalar(f"expert_load/{n}/{e}", v, ctx.global_step)
        if snap:
            self.loads.append(snap)
            if self.dump_dir:
                import numpy as np
                os.makedirs(self.dump_dir, exist_ok=True)
                for idx, name in enumerate(sorted(snap)):
                    m = re.search(r"layers\.(\d+)\.", name)
                    layer = int(m.group(1)) if m else idx
                    np.save(os.path.join(self.dump_dir, f"layer-{layer}-step{ctx.global_step}.npy"),
                            np.asarray(snap[name], dtype=np.float32))
        if self.enabled and hasattr(model, "update_topk_bias"):
            model.update_topk_bias()


@_reg
class MoEDropRateCallback(Callback):
    """Fraction of token copies above expert capacity (``capacity_factor``) per MoE layer (:2339-2405)."""

    def __init__(self, expert_num: int, capacity_factor: float, num_layers: int = 0, mtp_depth: int = 0, **kwargs):
        self.E, self.cf = expert_num, capacity_factor
        self.rates: List[Dict[str, float]] = []

    def on_step_end(self, ctx):
        model = getattr(ctx.engine, "model", None)
        if model is None:
            return
        snap = {}
        for n, m in model.named_modules():
            counts = getattr(m, "last_tokens_per_expert", None)
            if counts is not None:
                c = counts.detach().float()
                cap = self.cf * c.sum() / self.E
                snap[n] = float((c - cap).clamp_min(0).sum() / c.sum().clamp_min(1))
        if snap:
            self.rates.append(snap)
            logger.info("moe drop rate: %s", {k: round(v, 4) for k, v in snap.items()})


@_reg
class ColdHotExpertMonitor(Callback):
    """Tracks the hottest experts per layer over a window; the list can drive expert replication at
    serving time (the reference broadcasts hot-expert weights, :1979-2172)."""

    def __init__(self, moe_config=None, hidden_size: int = 0, ffn_hidden_size: int = 0, expert_parallel: int = 1,
                 model_parallel: int = 1, save_checkpoint_steps: int = 1, update_step: int = 100, hot_expert_num: int = 1, **kwargs):
        self.update_step, self.k = max(1, update_step), hot_expert_num
        self.acc: Dict[str, torch.Tensor] = {}
        self.hot: Dict[str, List[int]] = {}

    def on_step_end(self, ctx):
        model = getattr(ctx.engine, "model", None)
        if model is None:
            return
        for n, m in model.named_modules():
            counts = getattr(m, "last_tokens_per_expert", None)
            if counts is not None:
                self.acc[n] = self.acc.get(n, 0) + counts.detach().float().cpu()
        if ctx.global_step % self.update_step == 0:
            self.hot = {n: c.topk(min(self.k, c.numel())).indices.tolist() for n, c in self.acc.items()}
            self.acc = {}


@_reg
class StressDetectCallBack(Callback):
    """Periodic hardware self-check: a fixed bf16 GEMM whose checksum must be bit-identical on every rank and
    across repeats. A mismatch is a silent-data-corruption suspect and stops the run (:2175-2238)."""

    def __init__(self, detection_interval: int = 0, num_detections: int = 1, dataset_size: int = 0, size: int = 1024, **kwargs):
        self.interval, self.repeats, self.size = detection_interval, max(1, num_detections), size
        self.results: List[bool] = []

    def check(self) -> bool:
        dev = "cuda" if torch.cuda.is_available() else "cpu"
        g = torch.Generator(device="cpu").manual_seed(1234)
        a = torch.randn(self.size, self.size, generator=g).to(dev, torch.bfloat16 if dev == "cuda" else torch.float32)
        sums = []
        for _ in range(self.repeats + 1):
            sums.append((a @ a.t()).float().sum().reshape(1))
        ok = all(torch.equal(sums[0], s) for s in sums[1:])
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            t = torch.cat([sums[0], -sums[0]])
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ok = ok and bool(t[0] == -t[1])
        return ok

    def on_step_end(self, ctx):
        if self.interval and ctx.global_step % self.interval == 0:
            ok = self.check()
            self.results.append(ok)
            if not ok:
                raise RuntimeError(f"stress detection found inconsistent results at step {ctx.global_step}")
            logger.info("stress detection passed at step %d", ctx.global_step)


@_reg
class StressTestModelMonitor(Callback):
    """Every ``interval_steps`` the training pauses and each rank trains a small fixed model for a few steps on fixed
    data; the per-step losses and the final gradient norm must agree on all ranks (same seed, same arithmetic), and a
    rank that deviates by more than ``compare_interval_steps``-step tolerance is reported as a hardware suspect.

    The reference spawns a side training job from a model directory and greps its logs for the global norm and loss of
    every rank (``callback.py:2408-2700``); here the side job runs in process on the rank's own device, which tests the
    same thing — the GEMM / attention / optimizer path of this GPU against the other GPUs — without a second launcher.
    ``stress_model_dir`` / ``stress_dataset_dir`` / ``stress_master_port`` are accepted for configuration parity."""

    def __init__(self, interval_steps: int = 10, stress_model_dir: Optional[str] = None,
                 stress_dataset_dir: Optional[str] = None, stress_master_port: int = 8338,
                 compare_interval_steps: Optional[int] = None, check_stresslog_interval_time: int = 60,
                 stress_steps: int = 4, hidden_size: int = 256, tolerance: float = 0.0, **kwargs):
        self.interval, self.steps, self.hidden, self.tol = interval_steps, max(1, stress_steps), hidden_size, tolerance
        self.model_dir, self.dataset_dir = stress_model_dir, stress_dataset_dir
        self.reports: List[dict] = []

    def run_stress_job(self) -> torch.Tensor:
        """Losses of the fixed job followed by the last gradient norm: ``[steps + 1]`` fp32 on the CPU."""
        dev = "cuda" if torch.cuda.is_available() else "cpu"
        dtype = torch.bfloat16 if dev == "cuda" else torch.float32
        state = torch.get_rng_state()
        cuda_state = torch.cuda.get_rng_state() if dev == "cuda" else None
        try:
            g = torch.Generator(device="cpu").manual_seed(20240229)
            H = self.hidden
            w1 = (torch.randn(H, 4 * H, generator=g) * 0.02).to(dev, dtype).requires_grad_(True)
            w2 = (torch.randn(4 * H, H, generator=g) * 0.02).to(dev, dtype).requires_grad_(True)
            x = torch.randn(512, H, generator=g).to(dev, dtype)
            y = torch.randn(512, H, generator=g).to(dev, dtype)
            out = []
            norm = torch.zeros(())
            for _ in range(self.steps):
                loss = ((torch.nn.functional.silu(x @ w1) @ w2 - y).float() ** 2).mean()
                gw1, gw2 = torch.autograd.grad(loss, (w1, w2))
                norm = (gw1.float().pow(2).sum() + gw2.float().pow(2).sum()).sqrt()
                with torch.no_grad():
                    w1 -= 0.1 * gw1
                    w2 -= 0.1 * gw2
                out.append(loss.detach().float().cpu())
            out.append(norm.detach().float().cpu())
            return torch.stack(out)
        finally:
            torch.set_rng_state(state)
            if cuda_state is not None:
                torch.cuda.set_rng_state(cuda_state)

    def compare(self, mine: torch.Tensor) -> dict:
        """All-gather the results; ``{"ok", "max_spread", "suspects": [ranks that differ from the median]}``."""
        import torch.distributed as dist
        if not (dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1):
            return {"ok": bool(torch.isfinite(mine).all()), "max_spread": 0.0, "suspects": []}
        dev = "cuda" if dist.get_backend() == "nccl" else "cpu"
        rows = [torch.empty_like(mine, device=dev) for _ in range(dist.get_world_size())]
        dist.all_gather(rows, mine.to(dev))
        table = torch.stack(rows).cpu()
        med = table.median(dim=0).values
        dev_per_rank = (table - med).abs().max(dim=1).values
        suspects = [r for r, d in enumerate(dev_per_rank.tolist()) if d > self.tol or d != d]
        return {"ok": not suspects, "max_spread": float(dev_per_rank.max()), "suspects": suspects}

    def on_step_end(self, ctx):
        if not self.interval or ctx.global_step % self.interval:
            return
        report = self.compare(self.run_stress_job())
        report["step"] = ctx.global_step
        self.reports.append(report)
        if report["ok"]:
            logger.info("stress test at step %d: all ranks agree", ctx.global_step)
        else:
            logger.error("stress test at step %d: ranks %s deviate (max spread %.3e)", ctx.global_step,
                         report["suspects"], report["max_spread"])
            raise RuntimeError(f"stress test found deviating ranks {report['suspects']} at step {ctx.global_step}")


@_reg
class SDCMonitor(Callback):
    """Silent-data-corruption watch: re-runs the forward of one fixed micro-batch every ``checksum_interval``
    steps in ``torch.no_grad`` and compares the loss across data-parallel replicas of the same model shard
    (they hold identical weights, so their losses must match bit for bit). The reference greps device logs
    and toggles a checksum mode of its matmuls (:2703-2878); the comparison across replicas is the part
    that carries over to this hardware."""

    def __init__(self, initial_step: int = 0, step_interval: int = 10, checksum_interval: int = 0, probe_batch=None, **kwargs):
        self.interval = checksum_interval or step_interval
        self.probe = probe_batch
        self.mismatches: List[int] = []

    def on_step_end(self, ctx):
        if not self.interval or ctx.global_step % self.interval or self.probe is None:
            return
        import torch.distributed as dist
        from ..parallel import parallel_state as ps
        model = ctx.engine.model
        with torch.no_grad():
            loss = model(self.probe["input_ids"], self.probe["labels"]).detach().float().reshape(1)
        if dist.is_available() and dist.is_initialized() and ps.get_data_parallel_world_size() > 1:
            t = torch.cat([loss, -loss])
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=ps.get_data_parallel_group())
            if bool(t[0] != -t[1]):
                self.mismatches.append(ctx.global_step)
                raise RuntimeError(f"SDC suspected: replicas disagree on the probe loss at step {ctx.global_step}")


@_reg
class GracefulExitCallback(Callback):
    """Stops cleanly (after saving) when ``<path>`` contains ``{"GracefulExit": 1}``; the file is polled
    between steps, so no kernel or collective is in flight when ranks leave (``wrapper/wrapper.py:272-273``)."""

    def __init__(self, graceful_exit_path: Optional[str] = None, poll_steps: int = 1, **kwargs):
        self.path = graceful_exit_path or os.path.join(get_output_root_path(), "graceful_exit.json")
        self.poll = max(1, poll_steps)

    def requested(self) -> bool:
        try:
            with open(self.path) as f:
                return bool(json.load(f).get("GracefulExit"))
        except (OSError, ValueError):
            return False

    def on_step_end(self, ctx):
        if ctx.global_step % self.poll:
            return
        flag = self.requested()
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            t = torch.tensor([int(flag)], device="cuda" if dist.get_backend() == "nccl" else "cpu")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            flag = bool(t.item())
        if flag:
            logger.warning("Graceful exit is triggered, stop training at step %d", ctx.global_step)
            ctx.request_stop, ctx.stop_reason = True, "graceful_exit"


@_reg
class StepPauseCallback(Callback):
    """Training step pause (the TSP role of the reference's fault-tolerance runtime, ``version_control.py:412``
    ``check_tsp_valid``): while ``<path>`` contains ``{"Pause": 1}`` every rank waits at a step boundary, with no
    kernel or collective in flight, until the file is cleared (or says ``{"Pause": 0}``) or ``max_pause_seconds`` have
    passed. The ranks agree on pausing and on resuming through one all-reduce per poll, so none runs ahead; the time
    spent is recorded in ``paused_seconds``. An operator can use it to hold a job while a neighbour is serviced."""

    def __init__(self, pause_path: Optional[str] = None, poll_steps: int = 1, poll_seconds: float = 1.0,
                 max_pause_seconds: float = 3600.0, **kwargs):
        self.path = pause_path or os.path.join(get_output_root_path(), "step_pause.json")
        self.poll, self.poll_seconds, self.max_pause = max(1, poll_steps), float(poll_seconds), float(max_pause_seconds)
        self.paused_seconds, self.pauses = 0.0, 0

    def requested(self) -> bool:
        try:
            with open(self.path) as f:
                return bool(json.load(f).get("Pause"))
        except (OSError, ValueError):
            return False

    @staticmethod
    def _agree(flag: bool) -> bool:
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            t = torch.tensor([int(flag)], device="cuda" if dist.get_backend() == "nccl" else "cpu")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return bool(t.item())
        return flag

    def on_step_end(self, ctx):
        if ctx.global_step % self.poll or not self._agree(self.requested()):
            return
        import time as _time
        logger.warning("step pause requested: holding at step %d", ctx.global_step)
        self.pauses += 1
        t0 = _time.time()
        while True:
            _time.sleep(self.poll_seconds)
            waited = _time.time() - t0
            # a rank keeps pausing while ANY rank still sees the request, and all give up together at the limit
            if not self._agree(self.requested() and waited < self.max_pause):
                break
        self.paused_seconds += _time.time() - t0
        logger.warning("step pause over after %.1f s, resuming at step %d", _time.time() - t0, ctx.global_step)


@_reg
class TrainFaultTolerance(Callback):
    """Host-side fault handling around the step loop (the reference delegates to MindIO TFT,
    ``trainer/base_trainer.py:1095-1125``): on an exception it calls ``ckpt_save_fn`` (try-to-persist) once
    and, for recoverable errors whose message starts with ``TREError``, asks the trainer to roll back by
    reloading the latest checkpoint through ``ckpt_load_fn`` and continuing."""

    def __init__(self, ckpt_save_fn: Optional[Callable] = None, ckpt_load_fn: Optional[Callable] = None,
                 max_rollbacks: int = 3, **kwargs):
        self.save_fn, self.load_fn, self.max_rollbacks = ckpt_save_fn, ckpt_load_fn, max_rollbacks
        self.rollbacks = 0

    def on_exception(self, ctx, exc):
        recoverable = isinstance(exc, RuntimeError) and str(exc).startswith("TREError")
        if recoverable and self.load_fn is not None and self.rollbacks < self.max_rollbacks:
            self.rollbacks += 1
            logger.warning("rolling back after %s (rollback %d)", exc, self.rollbacks)
            ctx.extras["rollback"] = self.load_fn(ctx)
            return
        if self.save_fn is not None:
            self.save_fn(ctx)


def build_callback(config=None, default_args: Optional[dict] = None, **kwargs):
    """Callback(s) from ``{"type": ...}`` dict(s) (``core/callback/build_callback.py:23``)."""
    if config is None:
        return None
    if isinstance(config, (list, tuple)):
        return [build_callback(c, default_args) for c in config]
    if isinstance(config, Callback):
        return config
    return MindFormerRegister.get_instance_from_cfg(dict(config), MindFormerModuleType.CALLBACK, default_args=default_args)


from .._submodules import alias_children as _alias_children  # noqa: E402

_alias_children(__name__, ['callback', 'build_callback'])
