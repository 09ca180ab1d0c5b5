"""Registered loss: masked (vocab-parallel) cross-entropy, reference ``core/loss/loss.py:159``."""
from ..parallel.layers.loss import CrossEntropyLoss as _CE, VocabParallelCrossEntropy
from ..tools.register import MindFormerModuleType, MindFormerRegister


@MindFormerRegister.register(MindFormerModuleType.LOSS)
class CrossEntropyLoss(_CE):
    """``loss = Σ(nll·mask) / (Σmask + eps)`` over logits ``[T, V(/tp)]`` and int labels ``[T]``."""

    def __init__(self, parallel_config=None, check_for_nan_in_loss_and_grad: bool = False,
                 calculate_per_token_loss: bool = False, seq_split_num: int = 1, eps_const: float = 1e-8, **unused):
        super().__init__(calculate_per_token_loss=calculate_per_token_loss, eps=eps_const)


def build_loss(config=None, default_args=None, **kwargs):
    cfg = dict(config or {"type": "CrossEntropyLoss"})
    cfg.update(kwargs)
    return MindFormerRegister.get_instance_from_cfg(cfg, MindFormerModuleType.LOSS, default_args=default_args)


__all__ = ["CrossEntropyLoss", "VocabParallelCrossEntropy", "build_loss"]


from .._submodules import alias_children as _alias_children  # noqa: E402

_alias_children(__name__, ['loss', 'build_loss'])
