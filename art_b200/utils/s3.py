"""S3 mirroring of model directories through the ``aws`` CLI (parity: reference
``src/art/utils/s3.py:25-300``).

All subprocess execution goes through :func:`_run`, which tests replace with a fake.
Layout: ``s3://{bucket}/[prefix/]{project}/models/{name}[/{step:04d}]`` and
``.../zipped-steps/{step:04d}.zip``.
"""
from __future__ import annotations

import asyncio
import os
import tempfile
import zipfile
from asyncio.subprocess import DEVNULL, PIPE

from ..errors import ForbiddenBucketCreationError
from .limit_concurrency import limit_concurrency
from .output_dirs import get_output_dir_from_model_properties, get_step_checkpoint_dir

__all__ = ("s3_sync", "S3SyncError", "build_s3_path", "build_s3_zipped_step_path", "ensure_bucket_exists",
           "pull_model_from_s3", "push_model_to_s3", "archive_and_presign_step_url")


class S3SyncError(RuntimeError):
    """The ``aws s3`` command exited with a non-zero status."""


async def _run(cmd: list[str], *, capture: bool = False, quiet: bool = True) -> tuple[int, str, str]:
    out = PIPE if capture else (DEVNULL if quiet else None)
    proc = await asyncio.create_subprocess_exec(*cmd, stdout=out, stderr=out)
    so, se = await proc.communicate()
    return proc.returncode or 0, (so or b"").decode(), (se or b"").decode()


def _bucket(s3_bucket: str | None) -> str:
    return s3_bucket if s3_bucket is not None else os.environ["BACKUP_BUCKET"]


def build_s3_path(*, model_name: str, project: str, step: int | None = None, s3_bucket: str | None = None,
                  prefix: str | None = None) -> str:
    pre = f"{prefix.strip('/')}/" if prefix else ""
    path = f"s3://{_bucket(s3_bucket)}/{pre}{project}/models/{model_name}"
    return path if step is None else f"{path}/{step:04d}"


def build_s3_zipped_step_path(*, model_name: str, project: str, step: int, s3_bucket: str | None = None,
                              prefix: str | None = None) -> str:
    base = build_s3_path(model_name=model_name, project=project, s3_bucket=s3_bucket, prefix=prefix)
    return f"{base}/zipped-steps/{step:04d}.zip"


def _aws(profile: str | None) -> list[str]:
    return ["aws"] + (["--profile", profile] if profile else [])


@limit_concurrency(1)
async def s3_sync(source: str, destination: str, *, profile: str | None = None, verbose: bool = False,
                  delete: bool = False) -> None:
    """``aws s3 sync`` for directories / prefixes, ``aws s3 cp`` when the source is a single file."""
    single_file = os.path.isfile(source)
    cmd = _aws(profile) + ["s3", "cp" if single_file else "sync"]
    if delete and not single_file:
        cmd.append("--delete")
    cmd += [source, destination]
    rc, _, _ = await _run(cmd, quiet=not verbose)
    if rc != 0:
        raise S3SyncError(f"{' '.join(cmd)} exited with status {rc}")


async def ensure_bucket_exists(s3_bucket: str | None = None, profile: str | None = None) -> None:
    bucket = _bucket(s3_bucket)
    rc, _, _ = await _run(_aws(profile) + ["s3api", "head-bucket", "--bucket", bucket])
    if rc == 0:
        return
    rc, _, _ = await _run(_aws(profile) + ["s3api", "create-bucket", "--bucket", bucket], quiet=False)
    if rc != 0:
        raise ForbiddenBucketCreationError(
            message=f"Failed to create bucket {bucket}. It may already exist and belong to another user, "
                    "or your credentials may be insufficient to create an S3 bucket.")


async def pull_model_from_s3(model_name: str, project: str, step: int | None = None, s3_bucket: str | None = None,
                             prefix: str | None = None, verbose: bool = False, delete: bool = False,
                             art_path: str | None = None) -> str:
    """Download the model directory (or one step of it); returns the local model directory."""
    model_dir = get_output_dir_from_model_properties(project=project, name=model_name, art_path=art_path)
    target = model_dir if step is None else get_step_checkpoint_dir(model_dir, step)
    os.makedirs(target, exist_ok=True)
    src = build_s3_path(model_name=model_name, project=project, step=step, s3_bucket=s3_bucket, prefix=prefix)
    await ensure_bucket_exists(s3_bucket)
    await s3_sync(src, target, verbose=verbose, delete=delete)
    return model_dir


async def push_model_to_s3(model_name: str, project: str, s3_bucket: str | None = None, prefix: str | None = None,
                           verbose: bool = False, delete: bool = False, art_path: str | None = None) -> None:
    model_dir = get_output_dir_from_model_properties(project=project, name=model_name, art_path=art_path)
    if not os.path.exists(model_dir):
        raise FileNotFoundError(f"Local model directory {model_dir} does not exist.")
    dst = build_s3_path(model_name=model_name, project=project, s3_bucket=s3_bucket, prefix=prefix)
    await s3_sync(model_dir, dst, verbose=verbose, delete=delete)


async def archive_and_presign_step_url(model_name: str, project: str, step: int, s3_bucket: str | None = None,
                                       prefix: str | None = None, verbose: bool = False, delete: bool = False,
                                       art_path: str | None = None) -> str:
    """Zip one step directory, upload it, and return a 1-hour presigned URL."""
    model_dir = get_output_dir_from_model_properties(project=project, name=model_name, art_path=art_path)
    step_dir = get_step_checkpoint_dir(model_dir, step)
    if not os.path.exists(step_dir):
        raise ValueError(f"Local step directory does not exist: {step_dir}")
    dst = build_s3_zipped_step_path(model_name=model_name, project=project, step=step, s3_bucket=s3_bucket, prefix=prefix)
    with tempfile.TemporaryDirectory() as tmp:
        archive = os.path.join(tmp, "model.zip")
        with zipfile.ZipFile(archive, "w", zipfile.ZIP_DEFLATED) as z:
            for root, _, files in os.walk(step_dir):
                for f in files:
                    full = os.path.join(root, f)
                    z.write(full, os.path.relpath(full, step_dir))
        await ensure_bucket_exists(s3_bucket)
        await s3_sync(archive, dst, verbose=verbose, delete=delete)
    rc, out, err = await _run(["aws", "s3", "presign", dst.removeprefix("s3://"), "--expires-in", "3600"], capture=True)
    if rc != 0:
        raise RuntimeError(f"Failed to generate presigned URL: {err}")
    return out.strip()
