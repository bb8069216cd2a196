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

from .. import dev
from ..backend import Backend
from . import utils
from .utils import SERVER_TASK, _sky

SERVER_COMMAND = "python -m art_b200.cli run --host 0.0.0.0 --port 7999"


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
                                 health_timeout: float = 600.0, health_get=None) -> "SkyPilotBackend":
        sky = _sky(sky_module)
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
        poll = 0.0 if sky_module is not None else 5.0     # a fake module answers at once
        attempts = max(1, int(health_timeout // max(poll, 5.0)))
        base_url = await utils.wait_for_art_server_to_start(cluster_name, sky, attempts=attempts, interval=poll,
                                                            get=health_get)
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
        return await utils.is_task_created(self._cluster_name, SERVER_TASK, self._sky)

    async def _endpoint(self, port: int) -> str:
        return await utils._endpoint(self._cluster_name, port, self._sky)

    async def register(self, model) -> None:
        """Registers the model with the server on the cluster (and says where its logs are)."""
        print("Registering model with server")
        print(f"To view logs, run: 'sky logs {self._cluster_name}'")
        await super().register(model)

    async def _prepare_backend_for_training(self, model, config: dev.OpenAIServerConfig | None) -> tuple[str, str]:
        """The completion server is reached through the cluster's public port-8000 endpoint."""
        _, api_key = await super()._prepare_backend_for_training(model, config)
        port = int(((config or {}).get("server_args", {}) or {}).get("port", 8000))
        return f"{await self._endpoint(port)}/v1", api_key

    async def down(self) -> None:
        await asyncio.to_thread(lambda: self._sky.down(cluster_name=self._cluster_name))


def stop_server(cluster_name: str = "art", sky_module: Any = None) -> None:
    """Blocking wrapper of :func:`art_b200.skypilot.stop_server.stop_server` (console helper)."""
    from .stop_server import stop_server as _stop

    asyncio.run(_stop(cluster_name, sky_module))
