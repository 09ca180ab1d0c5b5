"""One optimisation step: micro-batch loop (gradient accumulation), gradient reduction, clipping, update.

Counterpart of the reference's ``MFTrainOneStepCell`` / ``MFPipelineWithLossScaleCell``
(``wrapper/wrapper.py:103-292,479-673``): forward → backward → (unscale) → data-parallel reduce →
overflow / spike check → global-norm clip → optimizer, returning
``(loss, overflow, loss_scale, lr, global_norm)``. Gradients accumulate in the flat fp32 buffer across
micro-batches; the check and the clip happen inside the fused AdamW kernel from device scalars, so the
step launches without waiting for the host.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional

import torch

from .. import parallel_state as ps
from .optimizer import DistributedOptimizer


class TrainOneStep:
    """Forward + backward over the micro-batches of a step, gradient reduction, overflow / NaN check, global-norm
    clipping, optimizer step and loss-scale update (reference ``wrapper/wrapper.py:303`` ``MFTrainOneStepCell``).
    ``__call__(batch)`` returns ``{loss, global_norm, skipped, loss_scale}`` as device tensors."""

    def __init__(self, model: torch.nn.Module, optimizer: DistributedOptimizer, *, micro_batch_size: int = 1,
                 loss_scale: float = 1.0, forward_fn: Optional[Callable] = None):
        self.model, self.optimizer = model, optimizer
        self.micro_batch_size = micro_batch_size
        self.loss_scale = loss_scale
        self.forward_fn = forward_fn or (lambda m, b: m(b["input_ids"], b["labels"], b.get("loss_mask"),
                                                        b.get("position_ids"), actual_seq_len=b.get("actual_seq_len"))
                                         if b.get("actual_seq_len") is not None else
                                         m(b["input_ids"], b["labels"], b.get("loss_mask"), b.get("position_ids")))
        self._loss_acc = None

    def __call__(self, batch: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        """``batch`` holds this data-parallel rank's samples: ``input_ids``/``labels`` ``[n, S]`` (device tensors)."""
        model, opt = self.model, self.optimizer
        n = batch["input_ids"].shape[0]
        mbs = self.micro_batch_size
        if n % mbs:
            raise ValueError(f"local batch {n} is not a multiple of the micro batch size {mbs}")
        n_mb = n // mbs
        opt.zero_grad()
        total = torch.zeros((), dtype=torch.float32, device=batch["input_ids"].device)
        per_token = getattr(model, "config", None) is not None and getattr(model.config, "calculate_per_token_loss", False)
        den_total = torch.zeros_like(total)
        inv_den = None
        if per_token and "labels" in batch and batch["labels"] is not None:
            # the number of target tokens of the whole step is known before any forward pass (it is the model's own
            # mask rule applied to the batch): every micro-batch's numerator is divided by it ON THE DEVICE, so the
            # step needs no host read of the denominator
            cfg = model.config
            labels = batch["labels"]
            if batch.get("loss_mask") is not None:
                mask = batch["loss_mask"].to(torch.bool) & (labels != cfg.ignore_token_id)
            else:
                mask = (batch["input_ids"] != cfg.pad_token_id) & (labels != cfg.ignore_token_id)
            den_all = mask.sum().to(torch.float32)
            if ps.get_data_parallel_world_size(with_context_parallel=True) > 1:
                import torch.distributed as dist
                dist.all_reduce(den_all, group=ps.get_data_parallel_group(with_context_parallel=True))
            inv_den = 1.0 / (den_all + 1e-8)
        for i in range(n_mb):
            mb = {k: v[i * mbs:(i + 1) * mbs] for k, v in batch.items() if v is not None}
            if i == n_mb - 1 and hasattr(opt, "begin_grad_overlap"):
                opt.begin_grad_overlap()      # the last backward pass: layer gradients are reduced as they become final
            out = self.forward_fn(model, mb)
            if per_token:
                num, den = out
                (num * (self.loss_scale if inv_den is None else self.loss_scale * inv_den)).backward()
                total += num.detach()
                den_total += den.detach()
            else:
                (out * (self.loss_scale / n_mb)).backward()
                total += out.detach() / n_mb
        dp = ps.get_data_parallel_world_size(with_context_parallel=True)
        scale = 1.0 / (dp * self.loss_scale)
        if per_token and inv_den is not None:
            scale = 1.0 / self.loss_scale                     # the gradients already carry 1 / (target tokens of the step)
            total = total / (den_total + 1e-8)                # this rank's mean loss per target token (a device value)
        elif per_token:
            # no labels in the batch to count from: normalise by the denominators the model returned (one host read)
            import torch.distributed as dist
            if dp > 1:
                dist.all_reduce(den_total, group=ps.get_data_parallel_group(with_context_parallel=True))
            scale = float(1.0 / (den_total.item() * self.loss_scale + 1e-8))
            total = total / (den_total / dp + 1e-8)
        opt.step(grad_scale=scale)
        return {"loss": total, "global_norm": opt.global_norm(scale), "skipped": opt.skipped,
                "lr": opt.current_lr(), "loss_scale": self.loss_scale}
