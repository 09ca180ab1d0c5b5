"""Helpers of the checkpoint transformation tool (reference ``tools/ckpt_transform/utils.py``)."""
import os
import sys


def show_progress(progress: float, prefix: str = ""):
    """One-line progress bar on stdout; ``progress`` in [0, 1]."""
    progress = min(max(float(progress), 0.0), 1.0)
    width = 50
    done = int(width * progress)
    sys.stdout.write(f"\r{prefix}: [{'=' * done}{' ' * (width - done)}] {progress * 100:.2f}%")
    if progress >= 1.0:
        sys.stdout.write("\n")
    sys.stdout.flush()


def make_soft_link(soft_link: str, ckpt_file: str, target_is_directory: bool = False):
    """(Re)creates ``soft_link`` → ``ckpt_file``; an existing link is replaced, an existing real file is an error."""
    if os.path.islink(soft_link):
        os.remove(soft_link)
    elif os.path.exists(soft_link):
        raise FileExistsError(f"{soft_link} exists and is not a link")
    os.makedirs(os.path.dirname(os.path.abspath(soft_link)), exist_ok=True)
    os.symlink(os.path.abspath(ckpt_file), soft_link, target_is_directory=target_is_directory)


def check_path(path: str, info: str = "path"):
    if not isinstance(path, str) or not path:
        raise ValueError(f"{info} must be a non-empty string, got {path!r}")
    if not os.path.exists(path):
        raise FileNotFoundError(f"{info} {path} does not exist")
    return path


def check_rank_folders(path: str, rank_id: int) -> bool:
    """Whether ``path/rank_{rank_id}`` exists."""
    return os.path.isdir(os.path.join(path, f"rank_{rank_id}"))


def check_ckpt_file_exist(path: str) -> bool:
    """Whether the directory holds a checkpoint file (``.ckpt`` / ``.safetensors`` / ``.pt``)."""
    return os.path.isdir(path) and any(f.endswith((".ckpt", ".safetensors", ".pt")) for f in os.listdir(path))


def is_power_of_two(number: int) -> bool:
    return isinstance(number, int) and number > 0 and number & (number - 1) == 0
