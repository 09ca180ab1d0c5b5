"""Model-hub access without a network: a directory tree plays the hub.

The reference talks to the openMind hub (``mindformers/tools/hub/hub.py``: ``snapshot_download``, ``upload_folder``,
``create_repo``, ``PushToHubMixin``). Here ``$MFB200_HUB_ROOT`` (default ``~/.cache/mindformers_b200/hub``) holds one
directory per repository id; download resolves a repository to that directory, upload copies files into it. A
repository that is not there raises with the path that was looked up.
"""
from __future__ import annotations

import fnmatch
import os
import shutil
from typing import Iterable, List, Optional


def hub_root() -> str:
    return os.environ.get("MFB200_HUB_ROOT", os.path.join(os.path.expanduser("~"), ".cache", "mindformers_b200", "hub"))


def repo_dir(repo_id: str) -> str:
    if os.path.isabs(repo_id) or repo_id.startswith("."):
        return repo_id
    return os.path.join(hub_root(), *repo_id.split("/"))


def create_repo(repo_id: str, exist_ok: bool = True, **kwargs) -> str:
    path = repo_dir(repo_id)
    if os.path.isdir(path) and not exist_ok:
        raise FileExistsError(f"repository {repo_id} already exists at {path}")
    os.makedirs(path, exist_ok=True)
    return path


def _match(name: str, patterns: Optional[Iterable[str]]) -> bool:
    return patterns is None or any(fnmatch.fnmatch(name, p) for p in patterns)


def snapshot_download(repo_id: str, allow_patterns=None, ignore_patterns=None, local_dir: Optional[str] = None,
                      **kwargs) -> str:
    src = repo_dir(repo_id)
    if not os.path.isdir(src):
        raise FileNotFoundError(f"repository {repo_id!r} is not available offline (looked in {src}); "
                                f"place its files there or set MFB200_HUB_ROOT")
    if local_dir is None:
        return src
    for root, _, files in os.walk(src):
        for f in files:
            rel = os.path.relpath(os.path.join(root, f), src)
            if _match(rel, allow_patterns) and not (ignore_patterns and _match(rel, ignore_patterns)):
                dst = os.path.join(local_dir, rel)
                os.makedirs(os.path.dirname(dst), exist_ok=True)
                shutil.copy2(os.path.join(root, f), dst)
    return local_dir


def hf_hub_download(repo_id: str, filename: str, **kwargs) -> str:
    path = os.path.join(snapshot_download(repo_id), filename)
    if not os.path.isfile(path):
        raise FileNotFoundError(f"{filename} is not part of repository {repo_id}")
    return path


def upload_folder(repo_id: str, folder_path: str, path_in_repo: str = "", allow_patterns=None, ignore_patterns=None,
                  **kwargs) -> List[str]:
    dst_root = os.path.join(create_repo(repo_id), path_in_repo)
    copied = []
    for root, _, files in os.walk(folder_path):
        for f in files:
            rel = os.path.relpath(os.path.join(root, f), folder_path)
            if _match(rel, allow_patterns) and not (ignore_patterns and _match(rel, ignore_patterns)):
                dst = os.path.join(dst_root, rel)
                os.makedirs(os.path.dirname(dst), exist_ok=True)
                shutil.copy2(os.path.join(root, f), dst)
                copied.append(rel)
    return sorted(copied)


class PushToHubMixin:
    """``obj.push_to_hub(repo_id)`` = ``save_pretrained`` into a scratch directory + ``upload_folder``."""

    def push_to_hub(self, repo_id: str, working_dir: Optional[str] = None, **kwargs) -> List[str]:
        import tempfile
        with tempfile.TemporaryDirectory() as tmp:
            target = working_dir or tmp
            self.save_pretrained(target, **{k: v for k, v in kwargs.items() if k in ("max_shard_size", "hf_names")})
            return upload_folder(repo_id, target)
