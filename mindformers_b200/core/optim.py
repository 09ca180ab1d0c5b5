"""Optimizers exposed through the registry.

``AdamW`` / ``FusedAdamW`` are front-ends of the flat-buffer sharded optimizer
(``parallel/distributed/optimizer.py``, fused sm_100a kernel); their constructor follows the reference's
``core/optim/adamw.py`` / ``fused_adamw.py`` (``params, learning_rate, betas, eps, weight_decay``).
``CAME`` (``core/optim/came.py:194``) is implemented with plain PyTorch ops (factored second moment with
confidence-guided update); SGD/Adam/etc. of ``torch.optim`` are registered under their own names.
"""
from __future__ import annotations

from typing import Callable, Iterable, Optional, Union

import torch

from ..parallel.distributed.optimizer import DistributedOptimizer
from ..tools.register import MindFormerModuleType, MindFormerRegister


@MindFormerRegister.register(MindFormerModuleType.OPTIMIZER)
class AdamW(DistributedOptimizer):
    """``AdamW(model, learning_rate=..., betas=..., eps=..., weight_decay=...)``.

    The first argument is the model (the optimizer lays its parameters out in flat buffers); weight decay is
    skipped for 1-D parameters and biases, as in ``trainer/optimizer_grouped_parameters.py:29-96``.
    """

    def __init__(self, params, learning_rate: Union[float, Callable] = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.0, **kw):
        if not isinstance(params, torch.nn.Module):
            raise TypeError("AdamW expects the model (nn.Module) whose parameters it should manage")
        kw.pop("use_fused", None)
        super().__init__(params, learning_rate=learning_rate, betas=tuple(betas), eps=eps, weight_decay=weight_decay,
                         **kw)


@MindFormerRegister.register(MindFormerModuleType.OPTIMIZER)
class FusedAdamW(AdamW):
    """Same update; the name of the reference's single-op variant."""


@MindFormerRegister.register(MindFormerModuleType.OPTIMIZER)
class CAME(torch.optim.Optimizer):
    """Confidence-guided Adaptive Memory Efficient optimizer (factored second moments)."""

    def __init__(self, params, learning_rate: float = 2e-4, eps=(1e-30, 1e-16), clip_threshold: float = 1.0,
                 betas=(0.9, 0.999, 0.9999), weight_decay: float = 0.0):
        if isinstance(params, torch.nn.Module):
            params = [p for p in params.parameters() if p.requires_grad]
        super().__init__(params, dict(lr=learning_rate, eps=eps, clip_threshold=clip_threshold, betas=betas,
                                      weight_decay=weight_decay))

    @staticmethod
    def _rms(t):
        return t.norm(2) / (t.numel() ** 0.5)

    @staticmethod
    def _approx_sq(row, col):
        r = (row / row.mean(dim=-1, keepdim=True)).rsqrt_().unsqueeze(-1)
        c = col.unsqueeze(-2).rsqrt()
        return r * c

    @torch.no_grad()
    def step(self, closure=None):
        for group in self.param_groups:
            b1, b2, b3 = group["betas"]
            e1, e2 = group["eps"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                g = p.grad.float()
                st = self.state[p]
                factored = g.dim() >= 2
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(g)
                    if factored:
                        st["row"] = torch.zeros(g.shape[:-1], device=g.device)
                        st["col"] = torch.zeros(g.shape[:-2] + g.shape[-1:], device=g.device)
                        st["res_row"] = torch.zeros_like(st["row"])
                        st["res_col"] = torch.zeros_like(st["col"])
                    else:
                        st["sq"] = torch.zeros_like(g)
                st["step"] += 1
                upd = g * g + e1
                if factored:
                    st["row"].mul_(b2).add_(upd.mean(-1), alpha=1 - b2)
                    st["col"].mul_(b2).add_(upd.mean(-2), alpha=1 - b2)
                    u = self._approx_sq(st["row"], st["col"]) * g
                else:
                    st["sq"].mul_(b2).add_(upd, alpha=1 - b2)
                    u = st["sq"].rsqrt() * g
                u.div_((self._rms(u) / group["clip_threshold"]).clamp_(min=1.0))
                st["exp_avg"].mul_(b1).add_(u, alpha=1 - b1)
                if factored:
                    res = (u - st["exp_avg"]) ** 2 + e2
                    st["res_row"].mul_(b3).add_(res.mean(-1), alpha=1 - b3)
                    st["res_col"].mul_(b3).add_(res.mean(-2), alpha=1 - b3)
                    out = self._approx_sq(st["res_row"], st["res_col"]) * st["exp_avg"]
                else:
                    out = st["exp_avg"].clone()
                if group["weight_decay"]:
                    p.mul_(1 - group["lr"] * group["weight_decay"])
                p.add_(out.to(p.dtype), alpha=-group["lr"])


for _name in ("SGD", "Adam", "Adagrad", "RMSprop", "Adamax", "NAdam", "RAdam"):
    if hasattr(torch.optim, _name) and not MindFormerRegister.is_exist(MindFormerModuleType.OPTIMIZER, _name):
        MindFormerRegister.register_cls(getattr(torch.optim, _name), MindFormerModuleType.OPTIMIZER, alias=_name)


def get_optimizer_grouped_parameters(model: torch.nn.Module, weight_decay: float = 0.0, layer_scale: bool = False,
                                     layer_decay: float = 1.0):
    """Parameter groups with weight decay disabled for biases, norms and other 1-D tensors; optional
    layer-wise learning-rate decay (``lr_scale`` per group)."""
    layers = [int(n.split("layers.")[1].split(".")[0]) for n, _ in model.named_parameters() if "layers." in n]
    num_layers = (max(layers) + 1) if layers else 0
    groups = {}
    for n, p in model.named_parameters():
        if not p.requires_grad:
            continue
        no_decay = p.dim() <= 1 or n.endswith(".bias") or getattr(p, "no_weight_decay", False)
        scale = 1.0
        if layer_scale and num_layers:
            if "layers." in n:
                lid = int(n.split("layers.")[1].split(".")[0]) + 1
            elif "embedding" in n:
                lid = 0
            else:
                lid = num_layers + 1
            scale = layer_decay ** (num_layers + 1 - lid)
        key = (no_decay, scale)
        groups.setdefault(key, {"params": [], "weight_decay": 0.0 if no_decay else weight_decay, "lr_scale": scale})
        groups[key]["params"].append(p)
    return list(groups.values())


# the reference registers this optimizer as ``Came`` (``core/optim/came.py``); YAMLs written for it say ``type: Came``
Came = CAME
MindFormerRegister.register_cls(CAME, MindFormerModuleType.OPTIMIZER, alias="Came")


class ReplicatedOptimizer:
    """Runs any ``torch.optim`` style optimizer (``CAME``, ``SGD``, ...) behind the interface the train step expects
    from the sharded AdamW: ``zero_grad()``, ``step(grad_scale)``, ``global_norm()``, ``skipped``, ``current_lr()``,
    ``global_step``, ``named_states()``. State is replicated over the data-parallel group: gradients are all-reduced
    (NCCL / gloo), the global norm is taken over all model-parallel ranks with tensor-parallel replicas counted once,
    clipping follows ``core/clip_grad.py`` (``max_norm / (norm + 1e-6)`` when the norm exceeds ``max_norm``), and
    a non-finite norm skips the update. This is how the trainer honours ``optimizer.type`` other than AdamW."""

    def __init__(self, model: torch.nn.Module, inner: torch.optim.Optimizer, learning_rate, max_grad_norm: float = 1.0,
                 sequence_parallel: bool = False):
        import torch.distributed as dist
        from ..parallel import parallel_state as ps
        self._dist, self._ps = dist, ps
        self.model, self.inner, self.lr = model, inner, learning_rate
        self.max_grad_norm, self.sequence_parallel = max_grad_norm, sequence_parallel
        self.global_step = 0
        dev = next(model.parameters()).device
        self.skipped = torch.zeros(1, dtype=torch.int32, device=dev)
        self.sumsq = torch.zeros(1, dtype=torch.float32, device=dev)
        self._base_lrs = [g.get("lr", 0.0) for g in inner.param_groups]

    def zero_grad(self, set_to_none: bool = True):
        self.inner.zero_grad(set_to_none=True)

    def current_lr(self) -> float:
        return float(self.lr(self.global_step) if callable(self.lr) else self.lr)

    def step(self, grad_scale: float = 1.0):
        dist, ps = self._dist, self._ps
        multi = dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1
        dp_group = ps.get_data_parallel_group(with_context_parallel=True) if multi else None
        tp = ps.get_tensor_model_parallel_world_size()
        self.sumsq.zero_()
        for p in self.model.parameters():
            if p.grad is None:
                continue
            if multi and ps.get_data_parallel_world_size(with_context_parallel=True) > 1:
                dist.all_reduce(p.grad, group=dp_group)
            if multi and tp > 1 and self.sequence_parallel and getattr(p, "sequence_parallel", False):
                dist.all_reduce(p.grad, group=ps.get_tensor_model_parallel_group())
            p.grad.mul_(grad_scale)
            ss = p.grad.float().pow(2).sum()
            replicated = tp > 1 and not getattr(p, "tensor_model_parallel", False) and not getattr(p, "is_expert", False)
            self.sumsq += ss / tp if replicated else ss
        if multi:
            dist.all_reduce(self.sumsq, group=ps.get_world_group())
            dpw = ps.get_data_parallel_world_size(with_context_parallel=True)
            if dpw > 1:
                self.sumsq /= dpw               # data-parallel replicas hold the same (already reduced) gradients
        norm = float(self.sumsq.sqrt())
        self.global_step += 1
        bad = not (norm == norm and norm != float("inf"))
        self.skipped.fill_(int(bad))
        if bad:
            return self.sumsq
        if self.max_grad_norm > 0 and norm >= self.max_grad_norm:
            coef = self.max_grad_norm / (norm + 1e-6)
            for p in self.model.parameters():
                if p.grad is not None:
                    p.grad.mul_(coef)
        lr = self.current_lr()
        for g in self.inner.param_groups:
            g["lr"] = lr * g.get("lr_scale", 1.0)
        self.inner.step()
        return self.sumsq

    def global_norm(self, grad_scale: float = 1.0) -> torch.Tensor:
        return self.sumsq.sqrt()        # ``step`` scaled the gradients before taking the norm

    def named_states(self):
        names = {id(p): n for n, p in self.model.named_parameters()}
        out = {}
        for p, st in self.inner.state.items():
            for k, v in st.items():
                if torch.is_tensor(v):
                    out[f"{k}.{names.get(id(p), 'param')}"] = v
        return out

    def load_named_states(self, states, global_step=None, strict: bool = False, model_params=None):
        by_name = dict(self.model.named_parameters())
        for key, v in states.items():
            if key.startswith("__slice__."):
                continue
            k, _, pname = key.partition(".")
            p = by_name.get(pname)
            if p is not None:
                self.inner.state.setdefault(p, {})[k] = v.to(p.device)
        if global_step is not None:
            self.global_step = int(global_step)

    def state_norms(self):
        return {}


def build_optim(config: dict, default_args: Optional[dict] = None, model: Optional[torch.nn.Module] = None, **kwargs):
    """Instantiate the optimizer named by ``config['type']``; ``model`` is passed as ``params``."""
    cfg = dict(config or {})
    cfg.update(kwargs)
    args = dict(default_args or {})
    if model is not None:
        args.setdefault("params", model)
    target = MindFormerRegister.get_cls(MindFormerModuleType.OPTIMIZER, cfg["type"])
    if not issubclass(target, DistributedOptimizer) and isinstance(args.get("params"), torch.nn.Module):
        layer_scale, layer_decay = bool(cfg.pop("layer_scale", False)), float(cfg.pop("layer_decay", 1.0))
        if layer_scale or cfg.get("weight_decay"):
            # decay / no-decay groups (and a learning rate that decays from the top layer down with layer_scale)
            from ..trainer.optimizer_grouped_parameters import get_optimizer_grouped_parameters
            args["params"] = get_optimizer_grouped_parameters(args["params"], float(cfg.get("weight_decay") or 0.0),
                                                              layer_scale=layer_scale, layer_decay=layer_decay)
        else:
            args["params"] = [p for p in args["params"].parameters() if p.requires_grad]
        if "learning_rate" in cfg and target.__module__.startswith("torch.optim"):
            cfg["lr"] = cfg.pop("learning_rate")
    return MindFormerRegister.get_instance_from_cfg(cfg, MindFormerModuleType.OPTIMIZER, default_args=args)


from .._submodules import alias_children as _alias_children  # noqa: E402

_alias_children(__name__, ['adamw', 'build_optim', 'came', 'fused_adamw'])
