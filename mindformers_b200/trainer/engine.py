"""``TrainingEngine``: model + sharded optimizer + step function behind one call.

This is the object ``Trainer`` drives and the one a user calls for a custom loop::

    engine = TrainingEngine.from_model_config(model_cfg, parallel=dict(tensor_model_parallel_size=2, ...))
    loss = engine.train_step({"input_ids": pinned_ids, "labels": pinned_labels})   # host tensors in, float out

``train_step`` copies the batch host→device (asynchronously from pinned memory), runs the micro-batch
loop and the optimizer, and reads the loss back; ``train_step_device`` is the same without the copies.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional, Union

import torch

from ..models.presets import preset_is_mla
from ..parallel import parallel_state as ps
from ..parallel.distributed.optimizer import DistributedOptimizer
from ..parallel.distributed.train_step import TrainOneStep
from ..parallel.layers.gpt_model import GPTModel
from ..parallel.transformer_config_utils import convert_to_transformer_config


class PipelineChunks(torch.nn.Module):
    """The model chunks one pipeline rank owns (one, or ``pp_interleave_num`` with virtual stages) behind the
    interface the optimizer and the checkpoint code expect from a model: parameters and buffers are reported under
    the names they have in the unsplit model (layers carry global numbers, so chunks never collide)."""

    def __init__(self, chunks):
        super().__init__()
        self.chunks = torch.nn.ModuleList(chunks)
        self.config = chunks[0].config

    def named_parameters(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True):
        for ch in self.chunks:
            yield from ch.named_parameters(prefix=prefix, recurse=recurse, remove_duplicate=remove_duplicate)

    def named_buffers(self, prefix: str = "", recurse: bool = True, remove_duplicate: bool = True):
        for ch in self.chunks:
            yield from ch.named_buffers(prefix=prefix, recurse=recurse, remove_duplicate=remove_duplicate)

    def forward(self, *args, **kwargs):
        raise RuntimeError("a pipeline stage is run by the pipeline schedule (TrainingEngine.train_step), not called directly")

    def update_topk_bias(self):
        for ch in self.chunks:
            ch.update_topk_bias()


def build_pipeline_chunks(tcfg) -> "PipelineChunks":
    """This rank's chunks for ``pipeline_model_parallel_size`` > 1: chunk ``c`` of stage ``r`` embeds when it is the
    first chunk of the first stage and computes the loss when it is the last chunk of the last stage."""
    pp, rank = ps.get_pipeline_model_parallel_world_size(), ps.get_pipeline_model_parallel_rank()
    v = tcfg.virtual_pipeline_model_parallel_size or 1
    chunks = []
    for c in range(v):
        if v > 1:
            ps.set_virtual_pipeline_model_parallel_rank(c)
        chunks.append(GPTModel(tcfg, pre_process=(rank == 0 and c == 0), post_process=(rank == pp - 1 and c == v - 1),
                               vp_stage=c if v > 1 else None))
    if v > 1:
        ps.set_virtual_pipeline_model_parallel_rank(0)
    return PipelineChunks(chunks)


class TrainingEngine:
    """One model + distributed optimizer + train step behind ``train_step(batch) -> {loss, global_norm, ...}``: the unit
    that ``bench.py`` and the trainers drive (reference ``wrapper/wrapper.py`` ``MFTrainOneStepCell`` plus the model /
    optimizer construction of ``trainer/base_trainer.py``)."""

    def __init__(self, model: torch.nn.Module, optimizer: DistributedOptimizer, micro_batch_size: int = 1,
                 loss_scale: float = 1.0, forward_fn: Optional[Callable] = None, seq_split_num: int = 1):
        self.model = model
        self.optimizer = optimizer
        if isinstance(model, PipelineChunks) or int(seq_split_num or 1) > 1:
            # pipeline stages: 1F1B (interleaved when the rank owns several chunks) over NCCL point-to-point; with
            # seq_split_num > 1 the sequence pipeline (chunks of a sequence as pipeline units, keys / values carried)
            from ..parallel.pipeline import PipelineTrainStep
            chunks = list(model.chunks) if isinstance(model, PipelineChunks) else [model]
            self.step_fn = PipelineTrainStep(chunks, optimizer, micro_batch_size=micro_batch_size,
                                             loss_scale=loss_scale, seq_split_num=seq_split_num)
        else:
            self.step_fn = TrainOneStep(model, optimizer, micro_batch_size=micro_batch_size, loss_scale=loss_scale,
                                        forward_fn=forward_fn)
        self.device = next(model.parameters()).device
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    @classmethod
    def from_model_config(cls, model_config: dict, *, parallel: Optional[dict] = None, device=None,
                          learning_rate: Union[float, Callable] = 1e-4, betas=(0.9, 0.95), eps=1e-8,
                          weight_decay: float = 0.1, max_grad_norm: float = 1.0, micro_batch_size: int = 1,
                          seq_length: Optional[int] = None, dtype: str = "bfloat16", recompute=False,
                          grad_dtype=torch.float32, **extra):
        parallel = dict(parallel or {})
        cfgd = dict(model_config)
        cfgd.update(parallel)
        cfgd.setdefault("params_dtype", dtype)
        cfgd.setdefault("compute_dtype", dtype)
        if seq_length:
            cfgd["seq_length"] = seq_length
            cfgd["max_position_embeddings"] = max(seq_length, 1)
        cfgd["recompute"] = recompute
        cfgd.update(extra)
        tcfg = convert_to_transformer_config(cfgd, is_mla_model=preset_is_mla(cfgd))
        tcfg.device = device or ("cuda" if torch.cuda.is_available() else "cpu")
        if ps.model_parallel_is_initialized() and ps.get_pipeline_model_parallel_world_size() > 1:
            model = build_pipeline_chunks(tcfg)
        else:
            model = GPTModel(tcfg)
        opt = DistributedOptimizer(model, learning_rate=learning_rate, betas=betas, eps=eps, weight_decay=weight_decay,
                                   max_grad_norm=max_grad_norm, grad_dtype=grad_dtype,
                                   sequence_parallel=bool(tcfg.sequence_parallel))
        return cls(model, opt, micro_batch_size=micro_batch_size)

    def train_step_device(self, batch: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        self.model.train()
        return self.step_fn(batch)

    def train_step_full(self, host_batch: Dict[str, torch.Tensor]) -> Dict[str, float]:
        """Like ``train_step`` but returns ``loss``, ``lr``, ``global_norm`` and ``skipped`` as Python values (one
        device→host read of five scalars). The same read carries the kernels' status words: a bounded device wait
        that ran out raises ``DeviceWaitTimeout``; an expert-parallel receive-buffer overflow sets
        ``moe_rows_dropped`` (the buffers are grown before the next step and the trainer logs the event)."""
        dev_batch = {k: v.to(self.device, non_blocking=True) for k, v in host_batch.items()
                     if torch.is_tensor(v) and k in ("input_ids", "labels", "loss_mask", "position_ids", "actual_seq_len")}
        out = self.train_step_device(dev_batch)
        loss = out["loss"].float().reshape(())
        if ps.model_parallel_is_initialized() and ps.get_data_parallel_world_size(with_context_parallel=True) > 1:
            # the logged loss is the mean over the data-parallel replicas (each saw other samples)
            import torch.distributed as dist
            loss = loss.clone()
            dist.all_reduce(loss, group=ps.get_data_parallel_group(with_context_parallel=True))
            loss = loss / ps.get_data_parallel_world_size(with_context_parallel=True)
        vals = [loss, out["global_norm"].float().reshape(()), out["skipped"].float().reshape(())]
        if self.device.type == "cuda":
            from ..ops import _lib
            vals.extend(_lib.status_word(self.device).float().unbind(0))     # wait status, expert-parallel overflow
        packed = torch.stack(vals).cpu()
        res = {"loss": float(packed[0]), "global_norm": float(packed[1]), "skipped": bool(packed[2] > 0),
               "lr": float(out["lr"]), "moe_rows_dropped": False}
        if len(vals) > 3:
            from ..ops import _lib
            # a wait that ran out means a kernel of this step worked on partial data: do not train on
            _lib.raise_on_status(int(packed[3]), "in a training step")
            if int(packed[4]):
                res["moe_rows_dropped"] = True
        self.adapt_moe_capacity()
        return res

    def train_step(self, host_batch: Dict[str, torch.Tensor]) -> float:
        dev_batch = {}
        for k, v in host_batch.items():
            if v is None:
                continue
            dev_batch[k] = v.to(self.device, non_blocking=True)
            self.h2d_bytes = sum(t.numel() * t.element_size() for t in host_batch.values() if t is not None)
        out = self.train_step_device(dev_batch)
        loss = out["loss"].float().cpu()          # device→host read of the step's result
        self.d2h_bytes = loss.numel() * loss.element_size()
        self.adapt_moe_capacity()
        return float(loss)

    def adapt_moe_capacity(self) -> bool:
        """Grow the expert-parallel receive buffers if the last step overflowed them (collective, synchronising;
        a no-op without fused expert parallelism)."""
        from ..parallel import fused_moe
        if not fused_moe.MoEExchange._instances:
            return False
        return fused_moe.adapt_capacity()
