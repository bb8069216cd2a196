"""Backend base class = HTTP client of the ``art`` server (parity: reference
``src/art/backend.py:17-213``; protocol: ``src/art/cli.py:47-138``)."""
from __future__ import annotations

import json
from typing import TYPE_CHECKING, AsyncIterator

import httpx
from tqdm import auto as tqdm

from . import dev
from .trajectories import TrajectoryGroup
from .types import TrainConfig
from .utils.deploy_model import LoRADeploymentJob, LoRADeploymentProvider
from .utils.log_http_errors import log_http_errors

if TYPE_CHECKING:
    from .model import Model, TrainableModel


class Backend:
    def __init__(self, *, base_url: str = "http://0.0.0.0:7999") -> None:
        self._base_url = base_url
        self._client = httpx.AsyncClient(base_url=base_url)

    async def _post(self, route: str, *, timeout: float | None = 600, **kw) -> httpx.Response:
        r = await self._client.post(route, timeout=timeout, **kw)
        r.raise_for_status()
        return r

    async def close(self) -> None:
        """Shut down the remote backend's model services."""
        await self._post("/close", timeout=None)

    async def register(self, model: "Model") -> None:
        await self._post("/register", json=model.model_dump())

    async def _get_step(self, model: "TrainableModel") -> int:
        return (await self._post("/_get_step", json=model.model_dump())).json()

    async def _delete_checkpoints(self, model: "TrainableModel", benchmark: str, benchmark_smoothing: float) -> None:
        await self._post("/_delete_checkpoints", json=model.model_dump(),
                         params={"benchmark": benchmark, "benchmark_smoothing": benchmark_smoothing})

    async def _prepare_backend_for_training(self, model: "TrainableModel",
                                            config: dev.OpenAIServerConfig | None) -> tuple[str, str]:
        r = await self._post("/_prepare_backend_for_training", json={"model": model.model_dump(), "config": config})
        base_url, api_key = r.json()
        return base_url, api_key

    async def _log(self, model: "Model", trajectory_groups: list[TrajectoryGroup], split: str = "val") -> None:
        await self._post("/_log", timeout=None, json={
            "model": model.model_dump(),
            "trajectory_groups": [g.model_dump() for g in trajectory_groups],
            "split": split,
        })

    async def _train_model(self, model: "TrainableModel", trajectory_groups: list[TrajectoryGroup],
                           config: TrainConfig, dev_config: dev.TrainConfig, verbose: bool = False
                           ) -> AsyncIterator[dict[str, float]]:
        body = {
            "model": model.model_dump(),
            "trajectory_groups": [g.model_dump() for g in trajectory_groups],
            "config": config.model_dump(),
            "dev_config": dev_config,
            "verbose": verbose,
        }
        async with self._client.stream("POST", "/_train_model", json=body, timeout=None) as response:
            response.raise_for_status()
            bar = None
            async for line in response.aiter_lines():
                if not line.strip():
                    continue
                result = json.loads(line)
                if "error" in result and "num_gradient_steps" not in result:
                    raise RuntimeError(result["error"])
                yield result
                total = result.pop("num_gradient_steps", None)
                if bar is None:
                    bar = tqdm.tqdm(total=total, desc="train")
                bar.update(1)
                bar.set_postfix(result)
            if bar is not None:
                bar.close()

    @log_http_errors
    async def _experimental_pull_from_s3(self, model: "Model", *, s3_bucket: str | None = None,
                                         prefix: str | None = None, verbose: bool = False, delete: bool = False) -> None:
        await self._post("/_experimental_pull_from_s3", json={
            "model": model.model_dump(), "s3_bucket": s3_bucket, "prefix": prefix, "verbose": verbose, "delete": delete})

    @log_http_errors
    async def _experimental_push_to_s3(self, model: "Model", *, s3_bucket: str | None = None,
                                       prefix: str | None = None, verbose: bool = False, delete: bool = False) -> None:
        await self._post("/_experimental_push_to_s3", json={
            "model": model.model_dump(), "s3_bucket": s3_bucket, "prefix": prefix, "verbose": verbose, "delete": delete})

    @log_http_errors
    async def _experimental_deploy(self, deploy_to: LoRADeploymentProvider, model: "Model", step: int | None = None,
                                   s3_bucket: str | None = None, prefix: str | None = None, verbose: bool = False,
                                   pull_s3: bool = True, wait_for_completion: bool = True) -> LoRADeploymentJob:
        r = await self._post("/_experimental_deploy", json={
            "deploy_to": deploy_to, "model": model.model_dump(), "step": step, "s3_bucket": s3_bucket,
            "prefix": prefix, "verbose": verbose, "pull_s3": pull_s3, "wait_for_completion": wait_for_completion})
        return LoRADeploymentJob(**r.json())
