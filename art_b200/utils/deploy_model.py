"""Serverless LoRA deployment (Together) of a checkpoint step (parity: reference
``src/art/utils/deploy_model.py:23-278``).

HTTP goes through :func:`_request`, which tests replace; nothing here touches a GPU.
"""
from __future__ import annotations

import asyncio
import json
import os
import time
from enum import Enum
from typing import TYPE_CHECKING, Any

from pydantic import BaseModel

from ..errors import (LoRADeploymentTimedOutError, UnsupportedBaseModelDeploymentError,
                      UnsupportedLoRADeploymentProviderError)
from .get_model_step import get_model_step
from .output_dirs import get_default_art_path
from .s3 import archive_and_presign_step_url, pull_model_from_s3

if TYPE_CHECKING:
    from ..model import TrainableModel

TOGETHER_API = "https://api.together.xyz/v1"
TOGETHER_SUPPORTED_BASE_MODELS = [
    "meta-llama/Meta-Llama-3.1-8B-Instruct",
    "meta-llama/Meta-Llama-3.1-70B-Instruct",
    "Qwen/Qwen2.5-14B-Instruct",
    "Qwen/Qwen2.5-72B-Instruct",
]
POLL_SECONDS = 15.0
POLL_TIMEOUT_SECONDS = 300.0
_ALREADY_EXISTS = "409 Client Error: Conflict for url: https://api.together.ai/api/admin/entity/Model"


class LoRADeploymentProvider(str, Enum):
    TOGETHER = "together"


class LoRADeploymentJobStatus(str, Enum):
    QUEUED = "Queued"
    RUNNING = "Running"
    COMPLETE = "Complete"
    FAILED = "Failed"


class LoRADeploymentJob(BaseModel):
    status: LoRADeploymentJobStatus
    job_id: str
    model_name: str
    failure_reason: str | None


async def _request(method: str, url: str, body: dict | None = None) -> Any:
    import aiohttp

    if "TOGETHER_API_KEY" not in os.environ:
        raise ValueError("TOGETHER_API_KEY is not set, cannot deploy LoRA to Together")
    headers = {"Authorization": f"Bearer {os.environ['TOGETHER_API_KEY']}", "Content-Type": "application/json"}
    async with aiohttp.ClientSession(headers=headers) as session:
        async with session.request(method, url, json=body) as resp:
            resp.raise_for_status()
            return await resp.json()


def model_checkpoint_id(model: "TrainableModel", step: int) -> str:
    return f"{model.project}-{model.name}-{step}"


def convert_together_job_status(status: str, message: str | None = None) -> LoRADeploymentJobStatus:
    if status == "Error" and message and _ALREADY_EXISTS in message:
        return LoRADeploymentJobStatus.COMPLETE
    if status in ("Bad", "Error"):
        return LoRADeploymentJobStatus.FAILED
    if status == "Retry Queued":
        return LoRADeploymentJobStatus.QUEUED
    return LoRADeploymentJobStatus(status)


async def deploy_together(model: "TrainableModel", presigned_url: str, step: int, verbose: bool = False) -> dict[str, Any]:
    if model.base_model not in TOGETHER_SUPPORTED_BASE_MODELS:
        raise UnsupportedBaseModelDeploymentError(
            message=f"Base model {model.base_model} is not supported for serverless LoRA deployment by Together. "
                    f"Supported models: {TOGETHER_SUPPORTED_BASE_MODELS}")
    result = await _request("POST", f"{TOGETHER_API}/models", {
        "model_name": model_checkpoint_id(model, step),
        "model_source": presigned_url,
        "model_type": "adapter",
        "base_model": model.base_model,
        "description": f"Deployed from ART. Project: {model.project}. Model: {model.name}. Step: {step}",
    })
    if verbose:
        print(f"Successfully uploaded to Together: {result}")
    return result


async def find_existing_together_job_id(model: "TrainableModel", step: int) -> str | None:
    ident = model_checkpoint_id(model, step)
    jobs = (await _request("GET", f"{TOGETHER_API}/jobs"))["data"]
    for job in sorted(jobs, key=lambda j: j["updated_at"], reverse=True):
        if ident in job["args"]["modelName"]:
            return job["job_id"]
    return None


async def check_together_job_status(job_id: str, verbose: bool = False) -> LoRADeploymentJob:
    result = await _request("GET", f"{TOGETHER_API}/jobs/{job_id}")
    if verbose:
        print(f"Job status: {json.dumps(result, indent=4)}")
    last = result["status_updates"][-1] if result.get("status_updates") else {}
    job = LoRADeploymentJob(status=convert_together_job_status(result["status"], last.get("message")), job_id=job_id,
                            model_name=result["args"]["modelName"], failure_reason=result.get("failure_reason"))
    if job.status == LoRADeploymentJobStatus.FAILED:
        job.failure_reason = last.get("message")
    return job


async def wait_for_together_job(job_id: str, verbose: bool = False) -> LoRADeploymentJob:
    deadline = time.time() + POLL_TIMEOUT_SECONDS
    while time.time() < deadline:
        job = await check_together_job_status(job_id, verbose)
        if job.status in (LoRADeploymentJobStatus.COMPLETE, LoRADeploymentJobStatus.FAILED):
            return job
        await asyncio.sleep(POLL_SECONDS)
    raise LoRADeploymentTimedOutError(message=f"LoRA deployment timed out after 5 minutes. Job ID: {job_id}")


async def deploy_model(deploy_to: LoRADeploymentProvider, model: "TrainableModel", step: int | None = None,
                       s3_bucket: str | None = None, prefix: str | None = None, verbose: bool = False,
                       pull_s3: bool = True, wait_for_completion: bool = True,
                       art_path: str | None = None) -> LoRADeploymentJob:
    """Publish one checkpoint step as a hosted LoRA; re-uses a live job for the same step."""
    art_path = art_path or get_default_art_path()
    os.makedirs(art_path, exist_ok=True)
    if pull_s3:
        await pull_model_from_s3(model_name=model.name, project=model.project, step=step, s3_bucket=s3_bucket,
                                 prefix=prefix, verbose=verbose, art_path=art_path)
    if step is None:
        step = get_model_step(model, art_path)
    url = await archive_and_presign_step_url(model_name=model.name, project=model.project, step=step,
                                             s3_bucket=s3_bucket, prefix=prefix, verbose=verbose, art_path=art_path)
    if deploy_to != LoRADeploymentProvider.TOGETHER:
        raise UnsupportedLoRADeploymentProviderError(f"Unsupported deployment option: {deploy_to}")
    job_id = await find_existing_together_job_id(model, step)
    existing = await check_together_job_status(job_id, verbose=verbose) if job_id else None
    if existing is None or existing.status == LoRADeploymentJobStatus.FAILED:
        job_id = (await deploy_together(model=model, presigned_url=url, step=step, verbose=verbose))["data"]["job_id"]
    if wait_for_completion:
        return await wait_for_together_job(job_id, verbose=verbose)
    return await check_together_job_status(job_id, verbose=verbose)
