"""``BaseDataset`` and the dataset-config checks (reference ``dataset/base_dataset.py:26-107``, ``dataset/utils.py:20-60``)."""
import inspect
from collections.abc import Iterable

from ..dataset.causal_language_model_dataset import data_shard_info, ResumableShardSampler  # noqa: F401
from ..tools.register import MindFormerConfig


class BaseDataset:
    """Base of the task datasets: holds ``dataset_config``; ``check_dataset_config`` builds one from a constructor's
    keyword arguments when none was given (so ``Dataset(dataset_config=cfg)`` and ``Dataset(data_loader=..., ...)`` are
    the same call); ``shard_info`` returns ``(shard_id, num_shards)`` of this rank's data-parallel group."""

    def __init__(self, dataset_config: dict = None):
        self.dataset_config = dataset_config

    @classmethod
    def check_dataset_config(cls, dataset_config, params):
        if not dataset_config:
            params = dict(params)
            params.pop("dataset_config", None)
            params.pop("cls", None)
            kwargs = params.pop("kwargs", None) or {}
            params.update(kwargs)
            dataset_config = MindFormerConfig(**params)
        return dataset_config

    @classmethod
    def init_dataset_config(cls, dataset_config):
        """Seeds the host-side random generators that shuffling and augmentation draw from."""
        import random

        import numpy as np
        import torch
        seed = getattr(dataset_config, "seed", None)
        if seed is not None:
            random.seed(seed)
            np.random.seed(seed % (2 ** 32))
            torch.manual_seed(seed)

    @classmethod
    def shard_info(cls):
        return data_shard_info()


def check_dataset_config(config):
    """Copies the run-level settings a dataset needs into ``config.train_dataset`` / ``config.eval_dataset`` (seed,
    batch size, micro-batch count, profile / auto-tune switches) and attaches each to its ``*_dataset_task``."""
    def _fill(ds, do_eval):
        ds.do_eval = do_eval
        for key in ("seed", "auto_tune", "filepath_prefix", "autotune_per_step", "profile"):
            ds[key] = config.get(key)
        runner = config.get("runner_config") or {}
        ds.batch_size = runner.get("batch_size")
        if not do_eval:
            ds.micro_batch_num = (config.get("parallel_config") or {}).get("micro_batch_num", 1)
            if ds.get("mixup_op"):
                ds.mixup_op.num_classes = runner.get("num_classes")
        if ds.get("output_columns") is None:
            ds.output_columns = ds.get("input_columns")

    if config.get("train_dataset") is not None:
        _fill(config.train_dataset, False)
        if config.get("train_dataset_task") is not None:
            config.train_dataset_task.dataset_config = config.train_dataset
    if config.get("eval_dataset") is not None:
        _fill(config.eval_dataset, True)
        if config.get("eval_dataset_task") is not None:
            config.eval_dataset_task.dataset_config = config.eval_dataset


def is_generator_function(func) -> bool:
    return inspect.isfunction(func) and inspect.isgeneratorfunction(func)


def check_dataset_iterable(dataset) -> bool:
    """Whether ``dataset`` can feed a trainer: an iterable, an indexable object, or a generator function."""
    return isinstance(dataset, Iterable) or hasattr(dataset, "__getitem__") or is_generator_function(dataset)


__all__ = ["BaseDataset", "ResumableShardSampler", "check_dataset_config", "check_dataset_iterable", "data_shard_info",
           "is_generator_function"]
