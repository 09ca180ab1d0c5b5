"""Object-store paths for indexed datasets.

Reference: ``dataset/blended_datasets/utils_s3.py`` (``S3Config``, ``is_s3_path``, ``parse_s3_path``, ``object_exists``,
``_s3_download_file`` and the cached ``.idx`` download that ``indexed_dataset.py`` uses for ``s3://`` prefixes).

The path handling and the local cache are here; the transfer itself needs ``boto3``, which is imported on first use and
reported clearly when it is missing (there is no network on the build machines, so the transfer is exercised with a
stand-in client in the tests).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any, Optional, Tuple

S3_PREFIX = "s3://"


@dataclass
class S3Config:
    """``path_to_idx_cache``: local directory that ``.idx`` files are downloaded to; ``bin_chunk_nbytes``: size of the
    ranged reads that serve ``.bin`` data."""
    path_to_idx_cache: str
    bin_chunk_nbytes: int = 256 * 1024 * 1024


def is_s3_path(path: str) -> bool:
    return isinstance(path, str) and path.startswith(S3_PREFIX)


def parse_s3_path(path: str) -> Tuple[str, str]:
    """``s3://bucket/key/parts`` → ``("bucket", "key/parts")``."""
    if not is_s3_path(path):
        raise ValueError(f"{path!r} is not an s3:// path")
    rest = path[len(S3_PREFIX):]
    bucket, _, key = rest.partition("/")
    if not bucket:
        raise ValueError(f"{path!r} has no bucket")
    return bucket, key


def get_client(client: Optional[Any] = None):
    if client is not None:
        return client
    try:
        import boto3
    except ImportError as e:
        raise ImportError("reading s3:// dataset prefixes needs boto3, which is not installed; copy the .bin/.idx "
                          "files to a local directory or install boto3") from e
    return boto3.client("s3")


def object_exists(path: str, client: Optional[Any] = None) -> bool:
    bucket, key = parse_s3_path(path)
    try:
        get_client(client).head_object(Bucket=bucket, Key=key)
        return True
    except Exception:            # botocore's ClientError (404) or a stand-in's KeyError
        return False


def download_file(path: str, local_path: str, client: Optional[Any] = None) -> str:
    bucket, key = parse_s3_path(path)
    os.makedirs(os.path.dirname(local_path) or ".", exist_ok=True)
    tmp = local_path + ".part"
    get_client(client).download_file(bucket, key, tmp)
    os.replace(tmp, local_path)
    return local_path


def cached_index_path(idx_path: str, config: S3Config) -> str:
    bucket, key = parse_s3_path(idx_path)
    return os.path.join(config.path_to_idx_cache, bucket, key)


def maybe_download_index(idx_path: str, config: S3Config, client: Optional[Any] = None) -> str:
    """Local path of an ``.idx`` file: downloaded once into the cache when ``idx_path`` is an s3:// path."""
    if not is_s3_path(idx_path):
        return idx_path
    local = cached_index_path(idx_path, config)
    if not os.path.exists(local):
        download_file(idx_path, local, client)
    return local


def read_range(path: str, offset: int, nbytes: int, client: Optional[Any] = None) -> bytes:
    """``nbytes`` of an object from ``offset`` (a ranged GET): how ``.bin`` data is read without a local copy."""
    bucket, key = parse_s3_path(path)
    resp = get_client(client).get_object(Bucket=bucket, Key=key, Range=f"bytes={offset}-{offset + nbytes - 1}")
    body = resp["Body"]
    return body.read() if hasattr(body, "read") else bytes(body)
