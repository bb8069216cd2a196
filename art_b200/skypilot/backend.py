"""SkyPilotBackend: provision a GPU VM with SkyPilot, run the backend server there, then behave
as an HTTP :class:`Backend` pointed at it (parity: reference ``src/art/skypilot/backend.py:23-223``
and ``utils.py:10-93``).

SkyPilot is an optional dependency; every call into it goes through the ``sky`` module object
passed to / imported by :func:`_sky`, so the control flow is testable with a fake module.
"""
from __future__ import annotations

import asyncio
import os
from typing import Any

import httpx

from .. import dev
from ..backend import Backend

SERVER_TASK = "art_server"
SERVER_COMMAND = "python -m art_b200.cli run --host 0.0.0.0 --port 7999"


def _sky():
    try:
        import sky  # type: ignore

        return sky
    except ImportError as e:
        raise RuntimeError("SkyPilotBackend needs the `skypilot` package, which is not installed") from e


def _load_env_file(path: str) -> dict[str, str]:
    env: dict[str, str] = {}
    with open(path) as f:
        for line in f:
            line = line.strip()
            if not line or line.startswith("#") or "=" not in line:
                continue
            k, _, v = line.partition("=")
            env[k.strip()] = v.strip().strip('"').strip("'")
    return env


class SkyPilotBackend(Backend):
    _cluster_name: str
    _envs: dict[str, str]

    @classmethod
    async def initialize_cluster(cls, *, cluster_name: str = "art", gpu: str | None = None, resources: Any = None,
                                 art_version: str | None = None, env_path: str | None = None,
                                 force_restart: bool = False, sky_module: Any = None,
                                 health_timeout: float = 600.0) -> "SkyPilotBackend":
        sky = sky_module or _sky()
        self = cls.__new__(cls)
        self._cluster_name = cluster_name
        self._sky = sky
        self._envs = _load_env_file(env_path) if env_path else {}
        if gpu is None and resources is None:
            raise ValueError("Either gpu or resources must be provided")
        if resources is None:
            resources = sky.Resources(accelerators={gpu or "B200": 1}, ports=[])
        elif gpu is not None:
            resources = resources.copy(accelerators={gpu: 1})
        ports = list(getattr(resources, "ports", None) or [])
        resources = resources.copy(ports=ports + [p for p in ("7999", "8000") if p not in ports])

        status = await asyncio.to_thread(lambda: sky.status(cluster_names=[cluster_name]))
        if not status or status[0]["status"] != sky.ClusterStatus.UP:
            await self._launch_cluster(resources, art_version)
        running = await self._task_running()
        if running and force_restart:
            await asyncio.to_thread(lambda: sky.cancel(cluster_name=cluster_name, all=True))
            await asyncio.sleep(0 if sky_module is not None else 5)
            running = False
        if not running:
            task = sky.Task(name=SERVER_TASK, run=SERVER_COMMAND)
            if art_version is not None and os.path.exists(art_version):
                task.workdir = art_version
            task.update_envs(self._envs)
            await asyncio.to_thread(lambda: sky.exec(task=task, cluster_name=cluster_name, detach_run=True))
        base_url = await self._endpoint(7999)
        await self._wait_healthy(base_url, health_timeout)
        Backend.__init__(self, base_url=base_url)
        return self

    async def _launch_cluster(self, resources: Any, art_version: str | None) -> None:
        sky = self._sky
        setup = "python -m pip install --upgrade pip"
        if art_version is None or not os.path.exists(art_version):
            setup += f" && python -m pip install {art_version or 'art-b200'}"
        task = sky.Task(name="art-b200-setup", setup=setup)
        task.set_resources(resources)
        task.update_envs(self._envs)
        await asyncio.to_thread(lambda: sky.launch(task, cluster_name=self._cluster_name, retry_until_up=True))

    async def _task_running(self) -> bool:
        sky = self._sky
        queue = await asyncio.to_thread(lambda: sky.queue(self._cluster_name))
        return any(job.get("job_name") == SERVER_TASK and str(job.get("status", "")).endswith(("RUNNING", "PENDING", "SETTING_UP"))
                   for job in queue)

    async def _endpoint(self, port: int) -> str:
        sky = self._sky
        ep = await asyncio.to_thread(lambda: sky.endpoints(self._cluster_name, port))
        url = ep[port] if isinstance(ep, dict) and port in ep else (ep[str(port)] if isinstance(ep, dict) else ep)
        return url if str(url).startswith("http") else f"http://{url}"

    async def _wait_healthy(self, base_url: str, timeout: float) -> None:
        deadline = asyncio.get_running_loop().time() + timeout
        async with httpx.AsyncClient() as client:
            while True:
                try:
                    r = await client.get(f"{base_url}/healthcheck", timeout=5)
                    if r.status_code == 200:
                        return
                except httpx.HTTPError:
                    pass
                if asyncio.get_running_loop().time() > deadline:
                    raise TimeoutError(f"backend server at {base_url} did not become healthy")
                await asyncio.sleep(2)

    async def _prepare_backend_for_training(self, model, config: dev.OpenAIServerConfig | None) -> tuple[str, str]:
        """The completion server is reached through the cluster's public port-8000 endpoint."""
        _, api_key = await super()._prepare_backend_for_training(model, config)
        port = int(((config or {}).get("server_args", {}) or {}).get("port", 8000))
        return f"{await self._endpoint(port)}/v1", api_key

    async def down(self) -> None:
        await asyncio.to_thread(lambda: self._sky.down(cluster_name=self._cluster_name))


def stop_server(cluster_name: str = "art", sky_module: Any = None) -> None:
    """Cancel the backend server task on the cluster (console helper)."""
    sky = sky_module or _sky()
    sky.cancel(cluster_name=cluster_name, all=True)
