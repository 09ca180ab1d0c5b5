"""Static catalogue of what the package supports (``mindformers/mindformer_book.py:59``)."""
from __future__ import annotations

import os
from collections import OrderedDict

from .models.presets import PRESETS


class MindFormerBook:
    """Static catalogue of what the framework supports: trainers and pipelines per task, models per family, and the
    project paths (reference ``mindformers/mindformer_book.py:59``)."""

    _PROJECT_PATH = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    _TRAINER_SUPPORT_TASKS_LIST = OrderedDict([
        ("general", ["common"]),
        ("text_generation", sorted(PRESETS)),
        ("multi_modal_to_text_generation", ["common"]),
    ])
    _PIPELINE_SUPPORT_TASK_LIST = OrderedDict([("text_generation", sorted(PRESETS)), ("multi_modal_to_text_generation", ["common"])])
    _MODEL_SUPPORT_LIST = OrderedDict([
        ("llama", ["llama2_7b", "llama3_1_8b", "llama3_1_70b"]), ("qwen2", ["qwen2_5_7b"]), ("qwen3", ["qwen3_8b", "qwen3_32b"]),
        ("qwen3_moe", ["qwen3_30b_a3b"]), ("deepseek_v3", ["deepseek_v3"]), ("deepseek_v2", ["deepseek_v2_236b"]),
        ("qwen2_moe", ["qwen1_5_moe_a2_7b"]), ("mixtral", ["mixtral_8x7b"]),
        ("telechat", ["telechat2_7b"]), ("glm", ["glm4_9b"]),
    ])

    @classmethod
    def get_project_path(cls):
        return cls._PROJECT_PATH

    @classmethod
    def get_trainer_support_task_list(cls):
        return cls._TRAINER_SUPPORT_TASKS_LIST

    @classmethod
    def get_pipeline_support_task_list(cls):
        return cls._PIPELINE_SUPPORT_TASK_LIST

    @classmethod
    def get_model_support_list(cls):
        return cls._MODEL_SUPPORT_LIST

    @classmethod
    def show_model_support_list(cls):
        for fam, names in cls._MODEL_SUPPORT_LIST.items():
            print(f"{fam}: {', '.join(names)}")

    @classmethod
    def get_default_checkpoint_download_folder(cls):
        return os.path.join(os.path.expanduser("~"), ".cache", "mindformers_b200", "checkpoint_download")
