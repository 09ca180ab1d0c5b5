"""Task trainer: builds dataset / network / optimizer / callbacks from a configuration and runs the loops.

Counterpart of ``mindformers/trainer/base_trainer.py`` (``training_process`` :882-1214, ``evaluate_process``
:1216, ``predict_process`` :1290) and ``trainer/causal_language_modeling/causal_language_modeling.py:47-439``.
Where the reference compiles one graph per step and sinks it to the device, this loop launches the step's
kernels asynchronously and reads the loss back once per step (the read is what ``MFLossMonitor`` prints);
step time comes from CUDA events on the compute stream.
"""
from __future__ import annotations

import os
import time
from typing import Any, Dict, List, Optional

import torch

from ..checkpoint.io import load_checkpoint
from ..core.callback import (Callback, CheckpointMonitor, EvalCallBack, GracefulExitCallback, MFLossMonitor, ProfileMonitor,
                             RunContext, TrainingStateMonitor, build_callback)
from ..core.lr import build_lr
from ..core.metric import build_metric
from ..dataset import build_dataset
from ..models import build_network
from ..parallel import parallel_state as ps
from ..tools.check_rules import check_rules
from ..tools.logger import get_logger
from ..tools.register.config import MindFormerConfig
from ..tools.register.register import MindFormerModuleType, MindFormerRegister
from ..tools.utils import get_output_root_path, get_real_group_size
from .engine import TrainingEngine

logger = get_logger()


def _model_dict(config) -> dict:
    model = config.get("model") or {}
    mc = dict(model.get("model_config") or {})
    arch = (model.get("arch") or {}).get("type")
    if arch and "architectures" not in mc:
        mc["architectures"] = [arch]
    mc.pop("type", None)
    from ..models import merge_moe_config
    # the older YAMLs describe the experts in a top-level ``moe_config`` section
    return merge_moe_config(mc, mc.pop("moe_config", None) or config.get("moe_config"))


def parallel_kwargs(config) -> dict:
    """YAML ``parallel_config`` → model-parallel fields of the transformer configuration."""
    pc = dict(config.get("parallel_config") or {})
    tp = int(pc.get("model_parallel", 1) or 1)
    out = dict(tensor_model_parallel_size=tp, pipeline_model_parallel_size=int(pc.get("pipeline_stage", 1) or 1),
               context_parallel_size=int(pc.get("context_parallel", 1) or 1),
               expert_model_parallel_size=int(pc.get("expert_parallel", 1) or 1),
               sequence_parallel=bool(pc.get("use_seq_parallel")) and tp > 1)
    algo = pc.get("context_parallel_algo")
    if algo:
        out["context_parallel_algo"] = algo
    if pc.get("ulysses_degree_in_cp"):
        out["ulysses_degree_in_cp"] = pc["ulysses_degree_in_cp"]
    if (pc.get("pp_interleave_num") or 1) > 1:
        out["virtual_pipeline_model_parallel_size"] = pc["pp_interleave_num"]
    return out


class BaseTrainer:
    """Builds the pieces and owns the loops; task trainers override ``forward_batch`` where they differ."""

    task = "general"

    def __init__(self, task: Optional[str] = None, model_name: Optional[str] = None):
        self.task_name, self.model_name = task or self.task, model_name
        self.config = None
        self.engine: Optional[TrainingEngine] = None
        self.callbacks: List[Callback] = []
        self.loss_history: List[float] = []

    # ------------------------------------------------------------------ global batch bookkeeping
    @staticmethod
    def global_batch_size(config) -> int:
        rc, pc = config.get("runner_config") or {}, config.get("parallel_config") or {}
        bs = int(rc.get("batch_size", 1))
        if ps.model_parallel_is_initialized():
            dp = ps.get_data_parallel_world_size()
        else:
            dp = int(pc.get("data_parallel", 1) or 1) if config.get("use_parallel") else 1
        pp = int(pc.get("pipeline_stage", 1) or 1)
        interleave = int(config.get("micro_batch_interleave_num", 1) or 1)
        if pp > 1:
            return bs * dp * int(pc.get("micro_batch_num", 1) or 1) * interleave
        return bs * dp * interleave * int(rc.get("gradient_accumulation_steps", 1) or 1)

    # ------------------------------------------------------------------ builders
    def create_dataset(self, config, which: str = "train"):
        task_cfg = config.get(f"{which}_dataset_task")
        ds_cfg = dict(config.get(f"{which}_dataset") or {})
        if not task_cfg:
            task_cfg = {"type": "CausalLanguageModelDataset"}
        task_cfg = dict(task_cfg)
        inner = dict(task_cfg.get("dataset_config") or {})
        inner.update(ds_cfg)
        rc = config.get("runner_config") or {}
        accum = int(rc.get("gradient_accumulation_steps", 1) or 1)
        micro = int((config.get("parallel_config") or {}).get("micro_batch_num", 1) or 1)
        pp = int((config.get("parallel_config") or {}).get("pipeline_stage", 1) or 1)
        interleave = int(config.get("micro_batch_interleave_num", 1) or 1)
        per_step = int(rc.get("batch_size", 1)) * (micro if pp > 1 else accum) * (interleave if pp == 1 else 1)
        inner["batch_size"] = per_step if which == "train" else int(rc.get("batch_size", 1))
        loader = inner.get("data_loader")
        if isinstance(loader, dict) and loader.get("type") == "MockDataLoader":
            mc = _model_dict(config)
            loader.setdefault("seq_length", mc.get("seq_length", 2048))
            loader.setdefault("vocab_size", mc.get("vocab_size", 32000))
        task_cfg["dataset_config"] = inner
        return build_dataset(task_cfg)

    def create_engine(self, config, total_steps: int, model=None) -> TrainingEngine:
        opt_cfg = dict(config.get("optimizer") or {"type": "AdamW"})
        lr_cfg = dict(config.get("lr_schedule") or {})
        lr = opt_cfg.get("learning_rate", 5e-5)
        if lr_cfg.get("type"):
            lr_cfg.setdefault("learning_rate", lr)
            if lr_cfg.get("total_steps", -1) in (-1, None):
                lr_cfg["total_steps"] = total_steps
            lr = build_lr(lr_cfg)
        wrapper = dict(config.get("runner_wrapper") or {})
        clip = wrapper.get("use_clip_grad", True)
        max_norm = float(wrapper.get("max_grad_norm", 1.0)) if clip else 0.0
        scale = wrapper.get("scale_sense", 1.0)
        loss_scale = float(scale) if isinstance(scale, (int, float)) else 1.0   # bf16 needs no dynamic scaling
        rc = config.get("runner_config") or {}
        mc = _model_dict(config)
        rcfg = dict(config.get("recompute_config") or {})
        recompute = rcfg.get("recompute") or False          # bool, or layers per pipeline stage
        skip = float(wrapper.get("global_norm_spike_threshold", 0) or 0) if wrapper.get("use_skip_data_by_global_norm") else 0.0
        pc = config.get("parallel_config") or {}
        seq_split = int(pc.get("seq_split_num", 1) or 1)
        if seq_split > 1 and int(pc.get("pp_interleave_num", 1) or 1) > 1:
            raise NotImplementedError("seq_split_num > 1 (sequence pipeline) cannot be combined with pp_interleave_num > 1")
        interleave = int(config.get("micro_batch_interleave_num", 1) or 1)
        pp = int(pc.get("pipeline_stage", 1) or 1)
        if interleave > 1 and pp > 1:
            raise NotImplementedError("micro_batch_interleave_num > 1 cannot be combined with pipeline_stage > 1: the "
                                      "pipeline schedule already keeps several micro-batches in flight")
        opt_type = str(opt_cfg.get("type", "AdamW"))
        sharded_adamw = opt_type.lower() in ("adamw", "fusedadamw", "fused_adamw", "adam_w")
        betas = tuple(opt_cfg.get("betas", (0.9, 0.999)))
        mbs = int(rc.get("batch_size", 1))
        if model is not None:
            if pp > 1:
                raise NotImplementedError("pipeline_stage > 1 needs the model built from the configuration (one chunk per "
                                          "stage); a ready-made network cannot be split")
            tcfg = model.config if hasattr(model.config, "sequence_parallel") else model.model.config
            net = model if hasattr(model.config, "sequence_parallel") else model.model
        else:
            from ..models.presets import preset_is_mla
            from ..parallel.layers.gpt_model import GPTModel
            from ..parallel.transformer_config_utils import convert_to_transformer_config
            from .engine import build_pipeline_chunks
            cfgd = dict(mc)
            cfgd.update(parallel_kwargs(config))
            dtype = mc.get("compute_dtype", "bfloat16") if torch.cuda.is_available() else mc.get("compute_dtype", "float32")
            cfgd.setdefault("params_dtype", dtype)
            cfgd.setdefault("compute_dtype", dtype)
            cfgd["recompute"] = recompute
            for key in ("select_recompute", "recompute_slice_activation", "select_comm_recompute",
                        "parallel_optimizer_comm_recompute"):
                if rcfg.get(key):
                    cfgd[key] = rcfg[key]
            swap = dict(config.get("swap_config") or {})
            if swap.get("swap"):
                cfgd.update(cpu_offloading=True, cpu_offloading_num_layers=swap.get("layer_swap"),
                            default_prefetch=int(swap.get("default_prefetch", 1) or 1))
            tcfg = convert_to_transformer_config(cfgd, is_mla_model=preset_is_mla(cfgd))
            tcfg.device = "cuda" if torch.cuda.is_available() else "cpu"
            net = build_pipeline_chunks(tcfg) if (pp > 1 and ps.model_parallel_is_initialized()
                                                  and ps.get_pipeline_model_parallel_world_size() > 1) else GPTModel(tcfg)
        if sharded_adamw:
            from ..parallel.distributed.optimizer import DistributedOptimizer
            opt = DistributedOptimizer(net, learning_rate=lr, betas=betas, eps=opt_cfg.get("eps", 1e-8),
                                       weight_decay=opt_cfg.get("weight_decay", 0.0), max_grad_norm=max_norm,
                                       skip_threshold=skip, sequence_parallel=bool(tcfg.sequence_parallel))
        else:
            # any other registered optimizer (CAME, SGD, ...): replicated state, NCCL gradient all-reduce
            from ..core.optim import ReplicatedOptimizer, build_optim
            inner_cfg = {k: v for k, v in opt_cfg.items() if k not in ("learning_rate",)}
            inner_cfg["learning_rate"] = float(lr(1)) if callable(lr) else float(lr)
            inner = build_optim(inner_cfg, model=net)
            opt = ReplicatedOptimizer(net, inner, lr, max_grad_norm=max_norm, sequence_parallel=bool(tcfg.sequence_parallel))
        forward_fn = None
        if interleave > 1:
            from ..wrapper import MicroBatchInterleaved
            wrapped = MicroBatchInterleaved(net, interleave)
            forward_fn = lambda m, b: wrapped(b["input_ids"], b["labels"], b.get("loss_mask"), b.get("position_ids"))  # noqa: E731
            mbs *= interleave                        # one forward call now carries `interleave` copies of the micro-batch
        return TrainingEngine(net, opt, micro_batch_size=mbs, loss_scale=loss_scale, forward_fn=forward_fn,
                              seq_split_num=seq_split)

    def create_callbacks(self, config, default: Dict[str, Any]) -> List[Callback]:
        cbs: List[Callback] = []
        for c in config.get("callbacks") or [dict(type="MFLossMonitor")]:
            c = dict(c)
            if c.get("type") == "ObsMonitor":
                continue
            cbs.append(build_callback(c, default_args=None) if c["type"] not in ("MFLossMonitor", "CheckpointMonitor")
                       else build_callback(c, default_args={k: v for k, v in default.items()
                                                            if k in ("global_batch_size",)}))
        mon = config.get("monitor_config") or {}
        if mon.get("monitor_on"):
            cbs.append(TrainingStateMonitor(config=mon, global_batch_size=default.get("global_batch_size", 0)))
        if config.get("profile"):
            cbs.append(ProfileMonitor(start_step=config.get("profile_start_step", 1), stop_step=config.get("profile_stop_step", 10),
                                      profile_rank_ids=config.get("profile_rank_ids"), profile_pipeline=config.get("profile_pipeline", False),
                                      profile_memory=config.get("profile_memory", False), mstx=config.get("mstx", False),
                                      config=config.get("parallel_config")))
        if config.get("use_graceful_exit"):
            cbs.append(GracefulExitCallback((config.get("graceful_exit_config") or {}).get("graceful_exit_path")))
        # monitors first, checkpoint last: a checkpoint is written only after the step's checks passed
        cbs.sort(key=lambda c: isinstance(c, CheckpointMonitor))
        return cbs

    # ------------------------------------------------------------------ training
    def training_process(self, config, network=None, dataset=None, callbacks: Optional[List[Callback]] = None, **kwargs):
        self.config = config
        check_rules(config, mode="train")
        loader = dataset if dataset is not None else self.create_dataset(config, "train")
        rc = config.get("runner_config") or {}
        epochs = int(rc.get("epochs", 1))
        steps_per_epoch = len(loader)
        if int(rc.get("sink_size", -1) or -1) > 0 and rc.get("sink_mode") and rc.get("sink_size", 1) > 1:
            steps_per_epoch = min(steps_per_epoch, int(rc["sink_size"]))
        total_steps = epochs * steps_per_epoch
        stop_step = int(rc.get("stop_step", 0) or 0)
        if stop_step:
            total_steps = min(total_steps, stop_step)
        gbs = self.global_batch_size(config)
        self.engine = engine = self.create_engine(config, total_steps, model=network)
        if config.get("only_save_strategy"):
            # build the model under this job's layout, write its slicing description and stop: the files are the
            # destination strategy of an offline checkpoint transformation (reference trainer/base_trainer.py)
            from ..checkpoint.sharding import save_strategy
            from ..tools.utils import get_real_rank
            path = os.path.join(config.get("output_dir") or get_output_root_path(), "strategy",
                                f"ckpt_strategy_rank_{get_real_rank()}.json")
            save_strategy(engine.model, path)
            logger.info("only_save_strategy: wrote %s, no training", path)
            return {"strategy_file": path}
        seq_len = int(getattr(getattr(engine.model, "config", None), "seq_length", 0) or 0)
        ctx = RunContext(engine=engine, config=config, epochs=epochs, steps_per_epoch=steps_per_epoch, total_steps=total_steps,
                         global_batch_size=gbs, seq_length=seq_len)
        self.callbacks = cbs = list(callbacks) if callbacks is not None else self.create_callbacks(config, {"global_batch_size": gbs})
        start_epoch, start_step = self._maybe_load(config, engine, gbs, steps_per_epoch)
        ctx.global_step = start_epoch * steps_per_epoch + start_step
        if ctx.global_step and not config.get("ignore_data_skip") and hasattr(loader, "set_init_step"):
            skip = config.get("data_skip_steps")
            loader.set_init_step(int(skip) if skip is not None else start_step)
        for cb in cbs:
            cb.on_train_begin(ctx)
        use_cuda = torch.cuda.is_available() and engine.device.type == "cuda"
        try:
            for epoch in range(start_epoch, epochs):
                ctx.epoch = epoch
                if hasattr(loader, "shard_sampler"):
                    loader.shard_sampler.set_epoch(epoch)
                ctx.step_in_epoch = start_step if epoch == start_epoch else 0
                for batch in loader:
                    if ctx.step_in_epoch >= steps_per_epoch or ctx.global_step >= total_steps:
                        break
                    for cb in cbs:
                        cb.on_step_begin(ctx)
                    if use_cuda:
                        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        ev0.record()
                    t0 = time.perf_counter()
                    out = engine.train_step_full(batch)
                    if use_cuda:
                        ev1.record()
                        ev1.synchronize()
                        ctx.step_ms = ev0.elapsed_time(ev1)
                    else:
                        ctx.step_ms = (time.perf_counter() - t0) * 1e3
                    ctx.global_step += 1
                    ctx.step_in_epoch += 1
                    ctx.loss, ctx.lr, ctx.global_norm, ctx.skipped = out["loss"], out["lr"], out["global_norm"], out["skipped"]
                    if out.get("moe_rows_dropped"):
                        logger.warning("step %d: expert-parallel receive buffers overflowed and token rows were dropped; "
                                       "the buffers have been grown for the next step", ctx.global_step)
                    self.loss_history.append(ctx.loss)
                    for cb in cbs:
                        cb.on_step_end(ctx)
                    if ctx.request_stop:
                        break
                if ctx.request_stop or ctx.global_step >= total_steps:
                    break
                for cb in cbs:
                    cb.on_epoch_end(ctx)
        except BaseException as exc:
            for cb in cbs:
                cb.on_exception(ctx, exc)
            raise
        for cb in cbs:
            cb.on_train_end(ctx)
        return ctx

    def _maybe_load(self, config, engine, gbs, steps_per_epoch):
        path = config.get("load_checkpoint")
        resume = config.get("resume_training")
        start_epoch = start_step = 0
        if not path and config.get("pretrained_model_dir") and config.get("run_mode") == "finetune":
            path = config["pretrained_model_dir"]
        if not path:
            return 0, 0
        fam = _model_dict(config).get("model_type", "llama")
        from .utils import load_resume_context_from_checkpoint, transform_and_load_checkpoint
        if resume:
            scalars = transform_and_load_checkpoint(config, engine.model, engine.optimizer, path, family=fam, resume=True)
            ctx = load_resume_context_from_checkpoint(scalars, path, resume, gbs, steps_per_epoch)
            start_epoch, start_step = ctx["initial_epoch"], ctx["initial_step"]
            logger.info("resumed from %s at epoch %d step %d", path, start_epoch + 1, start_step)
        else:
            transform_and_load_checkpoint(config, engine.model, engine.optimizer, path, family=fam, resume=False)
        return start_epoch, start_step

    # ------------------------------------------------------------------ evaluation / prediction
    @torch.no_grad()
    def evaluate_process(self, config, network=None, dataset=None, metric=None, **kwargs):
        self.config = config
        loader = dataset if dataset is not None else self.create_dataset(config, "eval")
        model = network if network is not None else (self.engine.model if self.engine else build_network(config.get("model") or {}))
        if config.get("load_checkpoint") and network is None and self.engine is None:
            load_checkpoint(getattr(model, "model", model), config["load_checkpoint"], strict=False)
        metric = metric or build_metric(config.get("metric") or {"type": "PerplexityMetric"})
        metrics = metric if isinstance(metric, list) else [metric]
        for m in metrics:
            m.clear()
        model.eval()
        dev = next(model.parameters()).device
        for batch in loader:
            ids = batch["input_ids"].to(dev)
            labels = batch.get("labels")
            labels = labels.to(dev) if labels is not None else ids
            mask = batch.get("loss_mask")
            loss = model(ids, labels, mask.to(dev) if mask is not None else None)
            for m in metrics:
                m.update(loss)
        out = {}
        for m in metrics:
            out.update(m.eval())
        logger.info("evaluation: %s", out)
        return out

    @torch.no_grad()
    def predict_process(self, config, input_data=None, network=None, tokenizer=None, **kwargs):
        from ..models import build_tokenizer
        from ..pipeline import pipeline
        self.config = config
        model = network if network is not None else build_network(config.get("model") or {})
        path = config.get("load_checkpoint") or config.get("pretrained_model_dir")
        if path and network is None:
            model.load_weights(path, strict=False)
        if network is None and hasattr(model, "apply_quantization_config"):
            # ``model.model_config.quantization_config`` or a top-level ``quantization_config`` section of the YAML
            model.apply_quantization_config(config.get("quantization_config"))
        if tokenizer is None:
            tok_cfg = (config.get("processor") or {}).get("tokenizer")
            tokenizer = build_tokenizer(tok_cfg) if tok_cfg else build_tokenizer({"type": "ByteTokenizer"})
        pipe = pipeline(task="text_generation", model=model, tokenizer=tokenizer)
        data = input_data if input_data is not None else config.get("input_data")
        if isinstance(data, str) and os.path.isfile(data):
            with open(data) as f:
                data = [line.rstrip("\n") for line in f if line.strip()]
        gen_kw = {k: kwargs[k] for k in ("max_new_tokens", "max_length", "do_sample", "top_k", "top_p", "temperature",
                                          "repetition_penalty", "num_beams") if k in kwargs}
        result = pipe(data, batch_size=config.get("predict_batch_size") or 1, **gen_kw)
        save = config.get("save_file") or os.path.join(get_output_root_path(), "text_generation_result.txt")
        os.makedirs(os.path.dirname(save) or ".", exist_ok=True)
        with open(save, "w") as f:
            for r in result if isinstance(result, list) else [result]:
                f.write(str(r) + "\n")
        return result


@MindFormerRegister.register(MindFormerModuleType.TRAINER, search_names=["text_generation"])
class CausalLanguageModelingTrainer(BaseTrainer):
    """Task trainer for causal language models (reference
    ``trainer/causal_language_modeling/causal_language_modeling.py:47-439``): ``train``, ``evaluate`` (perplexity),
    ``generate_evaluate`` (generate then score) and ``predict``."""

    task = "text_generation"

    def train(self, config, **kw):
        return self.training_process(config, **kw)

    def evaluate(self, config, **kw):
        return self.evaluate_process(config, **kw)

    def predict(self, config, **kw):
        return self.predict_process(config, **kw)

    def generate_evaluate(self, config, network=None, dataset=None, metric=None, tokenizer=None, max_new_tokens: int = 32, **kw):
        """Generate from each prompt, then score the text against the reference answers (EM/F1, ROUGE ...)."""
        from ..core.metric import EmF1Metric
        model = network if network is not None else self.engine.model
        metric = metric or EmF1Metric()
        metric.clear()
        for batch in dataset:
            prompts, answers = batch["prompt"], batch["answer"]
            ids = [tokenizer.encode(p) for p in prompts]
            outs = model.generate(ids, max_new_tokens=max_new_tokens)
            texts = [tokenizer.decode(o[len(i):]) for o, i in zip(outs, ids)]
            metric.update(texts, answers)
        return metric.eval()


class GeneralEngine:
    """The minimum a training loop needs, around an arbitrary network: ``train_step_full(batch)`` → ``{loss, lr,
    global_norm, skipped}``. ``network(batch)`` (a mapping is passed as keyword arguments, a tuple as positional ones)
    returns the loss or a tuple whose first element is the loss. Either ``wrapper`` — a callable that does forward,
    backward and the update itself and returns the loss, the counterpart of a ``TrainOneStepCell`` handed to the
    reference's general trainer — or ``optimizer`` (any ``torch.optim.Optimizer``) drives the update."""

    def __init__(self, network: torch.nn.Module, optimizer=None, wrapper=None, max_grad_norm: float = 0.0,
                 lr_scheduler=None, device=None):
        self.model, self.optimizer, self.wrapper = network, optimizer, wrapper
        self.max_grad_norm, self.lr_scheduler = float(max_grad_norm or 0.0), lr_scheduler
        first = next(network.parameters(), None)
        self.device = device or (first.device if first is not None else torch.device("cpu"))
        self.global_step = 0

    def _to_device(self, batch):
        move = lambda t: t.to(self.device, non_blocking=True) if isinstance(t, torch.Tensor) else t   # noqa: E731
        if isinstance(batch, dict):
            return {k: move(v) for k, v in batch.items()}
        if isinstance(batch, (list, tuple)):
            return type(batch)(move(v) for v in batch)
        return move(batch)

    def forward(self, batch):
        batch = self._to_device(batch)
        out = self.model(**batch) if isinstance(batch, dict) else (self.model(*batch) if isinstance(batch, (list, tuple))
                                                                    else self.model(batch))
        return out

    @staticmethod
    def loss_of(out):
        return out[0] if isinstance(out, (list, tuple)) else out

    def train_step_full(self, batch):
        self.model.train()
        if self.wrapper is not None:
            loss = self.loss_of(self.wrapper(self._to_device(batch)))
            norm = float("nan")
        else:
            self.optimizer.zero_grad(set_to_none=True)
            loss = self.loss_of(self.forward(batch))
            loss.backward()
            params = [p for g in self.optimizer.param_groups for p in g["params"] if p.grad is not None]
            if self.max_grad_norm > 0:
                norm = float(torch.nn.utils.clip_grad_norm_(params, self.max_grad_norm))
            else:
                norm = float(torch.linalg.vector_norm(torch.stack([torch.linalg.vector_norm(p.grad.float())
                                                                   for p in params]))) if params else 0.0
            self.optimizer.step()
            if self.lr_scheduler is not None:
                self.lr_scheduler.step()
        self.global_step += 1
        lr = self.optimizer.param_groups[0]["lr"] if self.optimizer is not None else float("nan")
        return {"loss": float(loss.detach()), "lr": float(lr), "global_norm": norm, "skipped": False}


@MindFormerRegister.register(MindFormerModuleType.TRAINER, search_names=["general"])
class GeneralTaskTrainer(BaseTrainer):
    """Trainer for a task this package has no dedicated flow for (reference
    ``trainer/general_task_trainer/general_task_trainer.py:32-240``): the caller brings the network and the dataset —
    and optionally the optimizer, a one-step ``wrapper``, callbacks and metric objects — and gets the common loop
    (callbacks, step timing, stop step) around them. Unlike the language-model trainers nothing is built from the
    model section of the configuration, so a missing network or dataset is an error, as in the reference."""

    task = "general"

    def create_engine(self, config, total_steps: int, model=None):
        from ..core.optim import build_optim
        kw = getattr(self, "_general_kwargs", {})
        optimizer, wrapper = kw.get("optimizer"), kw.get("wrapper")
        if optimizer is None and wrapper is None:
            opt_cfg = dict((config or {}).get("optimizer") or {"type": "AdamW", "learning_rate": 1e-3})
            if opt_cfg.get("type") in ("AdamW", "adamw", "FusedAdamW"):        # the sharded optimizer needs a GPT-style model
                lr = float(opt_cfg.get("learning_rate", 1e-3))
                optimizer = torch.optim.AdamW([p for p in model.parameters() if p.requires_grad], lr=lr,
                                              betas=tuple(opt_cfg.get("betas", (0.9, 0.999))), eps=float(opt_cfg.get("eps", 1e-8)),
                                              weight_decay=float(opt_cfg.get("weight_decay", 0.0)))
            else:
                optimizer = build_optim(opt_cfg, model=model)
        wrap_cfg = dict((config or {}).get("runner_wrapper") or {})
        clip = float(wrap_cfg.get("max_grad_norm", 0.0)) if wrap_cfg.get("use_clip_grad") else 0.0
        return GeneralEngine(model, optimizer, wrapper, clip, kw.get("lr_scheduler"))

    def global_batch_size(self, config):
        return int(((config or {}).get("runner_config") or {}).get("batch_size", 1) or 1)

    def _maybe_load(self, config, engine, gbs, steps_per_epoch):
        path = (config or {}).get("load_checkpoint")
        if path:
            from safetensors.torch import load_file
            state = load_file(path) if str(path).endswith(".safetensors") else torch.load(path, map_location="cpu")
            engine.model.load_state_dict(state, strict=False)
        return 0, 0

    def train(self, config=None, network=None, dataset=None, wrapper=None, optimizer=None, callbacks=None, **kwargs):
        if network is None:
            raise NotImplementedError("the general trainer needs the network to train, got None")
        if dataset is None:
            raise NotImplementedError("the general trainer needs the training dataset, got None")
        self._general_kwargs = dict(optimizer=optimizer, wrapper=wrapper, lr_scheduler=kwargs.pop("lr_scheduler", None))
        cfg = config if config is not None else MindFormerConfig({"runner_config": {"epochs": 1}})
        if callbacks is None:
            callbacks = [MFLossMonitor()] if not (cfg.get("callbacks") or []) else None
        return self.training_process(cfg, network=network, dataset=dataset, callbacks=callbacks, **kwargs)

    @torch.no_grad()
    def evaluate(self, config=None, network=None, dataset=None, compute_metrics=None, callbacks=None, **kwargs):
        """``compute_metrics``: ``{name: metric}`` with ``clear()`` / ``update(*outputs)`` / ``eval()``; the network's
        evaluation output (a tensor or a tuple) is what ``update`` receives, batch by batch."""
        if network is None:
            raise NotImplementedError("the general trainer needs the network to evaluate, got None")
        if dataset is None:
            raise NotImplementedError("the general trainer needs the evaluation dataset, got None")
        if not compute_metrics:
            raise NotImplementedError("the general trainer needs compute_metrics = {name: metric object}")
        engine = GeneralEngine(network)
        network.eval()
        for m in compute_metrics.values():
            m.clear()
        for batch in dataset:
            out = engine.forward(batch)
            out = out if isinstance(out, (list, tuple)) else (out,)
            for m in compute_metrics.values():
                m.update(*out)
        result = {name: m.eval() for name, m in compute_metrics.items()}
        logger.info("evaluation: %s", result)
        return result

    @torch.no_grad()
    def predict(self, config=None, input_data=None, network=None, **kwargs):
        """Runs ``network`` in evaluation mode on ``input_data`` (one batch, or a list of batches) and returns its raw
        outputs: what a prediction *means* belongs to the task, which this trainer does not know."""
        if network is None:
            raise NotImplementedError("the general trainer needs the network to predict with, got None")
        engine = GeneralEngine(network)
        network.eval()
        if isinstance(input_data, list) and input_data and isinstance(input_data[0], (dict, tuple, list, torch.Tensor)):
            return [engine.forward(b) for b in input_data]
        return engine.forward(input_data)


@MindFormerRegister.register(MindFormerModuleType.TRAINER, search_names=["multi_modal_to_text_generation"])
class MultiModalToTextGenerationTrainer(CausalLanguageModelingTrainer):
    """Task trainer for image / multimodal-to-text models (reference
    ``trainer/multi_modal_to_text_generation/multi_modal_to_text_generation.py:35-260``): training and evaluation are
    the causal-LM flow on batches that also carry the modality tensors; ``predict`` turns conversation records
    (``[{"image": path}, {"text": ...}]`` per query) into tensors with the model's processor, generates and decodes."""

    task = "multi_modal_to_text_generation"

    def predict(self, config, input_data=None, network=None, tokenizer=None, processor=None, **kwargs):
        from ..models import build_processor, build_tokenizer
        from ..pipeline import pipeline
        self.config = config
        model = network if network is not None else build_network(config.get("model") or {})
        path = config.get("load_checkpoint") or config.get("pretrained_model_dir")
        if path and network is None:
            model.load_weights(path, strict=False)
        proc_cfg = config.get("processor") or {}
        if tokenizer is None:
            tok_cfg = proc_cfg.get("tokenizer")
            tokenizer = build_tokenizer(tok_cfg) if tok_cfg else build_tokenizer({"type": "ByteTokenizer"})
        if processor is None and proc_cfg.get("type"):
            processor = build_processor(proc_cfg, default_args={"tokenizer": tokenizer})
        data = input_data if input_data is not None else config.get("input_data")
        if isinstance(data, str) and os.path.isfile(data):
            import json as _json
            with open(data) as f:
                data = [_json.loads(line) for line in f if line.strip()]
        if isinstance(data, dict) or (isinstance(data, list) and data and isinstance(data[0], dict) and
                                      not any(isinstance(v, list) for v in data[0].values())):
            data = [data] if isinstance(data, dict) else [data]     # one query given as its list of segments
        pipe = pipeline(task="multi_modal_to_text_generation", model=model, tokenizer=tokenizer, processor=processor)
        gen_kw = {k: kwargs[k] for k in ("max_new_tokens", "max_length", "do_sample", "top_k", "top_p", "temperature",
                                          "repetition_penalty") if k in kwargs}
        result = pipe(data, batch_size=config.get("predict_batch_size") or 1, **gen_kw)
        save = config.get("save_file") or os.path.join(get_output_root_path(), "multi_modal_to_text_generation_result.txt")
        os.makedirs(os.path.dirname(save) or ".", exist_ok=True)
        with open(save, "w") as f:
            for r in result if isinstance(result, list) else [result]:
                f.write(str(r) + "\n")
        return result


def build_trainer(config: Optional[dict] = None, default_args=None, **kwargs):
    cfg = dict(config or {"type": "CausalLanguageModelingTrainer"})
    cfg.setdefault("type", "CausalLanguageModelingTrainer")
    cls = MindFormerRegister.get_cls(MindFormerModuleType.TRAINER, cfg["type"])
    return cls(task=cfg.get("task"), model_name=cfg.get("model_name"))
