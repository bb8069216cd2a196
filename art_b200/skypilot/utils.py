"""Polling helpers around a SkyPilot cluster: task state, start-up waits, endpoint lookup.

Parity: reference ``src/art/skypilot/utils.py:10-93`` (``get_task_status``, ``is_task_created``,
``wait_for_task_to_start``, ``wait_for_art_server_to_start``, ``get_art_server_base_url``,
``get_vllm_base_url``).  Differences: every function takes the ``sky`` module as an optional
argument (so the control flow runs against a fake in tests and SkyPilot stays an optional
dependency), poll interval and attempts are parameters, and the health wait raises when the
server never answers (the reference falls out of its loop silently).
"""
from __future__ import annotations

import asyncio
from typing import Any, Awaitable, Callable, TypeVar

import httpx

T = TypeVar("T")
SERVER_TASK = "art_server"
BACKEND_PORT = 7999
INFERENCE_PORT = 8000
# job states in which a task exists and may still (come to) run
_LIVE_STATES = ("INIT", "PENDING", "SETTING_UP", "RUNNING")


def _sky(sky_module: Any = None):
    if sky_module is not None:
        return sky_module
    try:
        import sky  # type: ignore

        return sky
    except ImportError as e:
        raise RuntimeError("this helper needs the `skypilot` package, which is not installed") from e


async def to_thread_typed(func: Callable[[], T]) -> T:
    return await asyncio.to_thread(func)


def _state_name(status: Any) -> str | None:
    """``sky.JobStatus.RUNNING`` / ``"JobStatus.RUNNING"`` / ``"RUNNING"`` -> ``"RUNNING"``."""
    if status is None:
        return None
    name = getattr(status, "name", None) or str(status)
    return name.rsplit(".", 1)[-1]


async def get_task_status(cluster_name: str, task_name: str, sky_module: Any = None) -> Any:
    """Status of the newest job called ``task_name`` in the cluster's queue, ``None`` if there is none."""
    sky = _sky(sky_module)
    queue = await to_thread_typed(lambda: sky.queue(cluster_name))
    for job in queue:
        if job.get("job_name") == task_name:
            return job.get("status")
    return None


async def is_task_created(cluster_name: str, task_name: str, sky_module: Any = None) -> bool:
    return _state_name(await get_task_status(cluster_name, task_name, sky_module)) in _LIVE_STATES


async def wait_for_task_to_start(cluster_name: str, task_name: str, sky_module: Any = None, *, attempts: int = 12,
                                 interval: float = 5.0) -> None:
    """Poll until the task is RUNNING (default: every 5 s for a minute)."""
    for _ in range(attempts):
        state = _state_name(await get_task_status(cluster_name, task_name, sky_module))
        if state is None:
            raise ValueError(f"Task {task_name} not found in cluster {cluster_name}")
        if state == "RUNNING":
            return
        if state not in _LIVE_STATES:
            raise ValueError(f"Task {task_name} in cluster {cluster_name} ended in state {state}")
        await asyncio.sleep(interval)
    raise ValueError(f"Task {task_name} in cluster {cluster_name} failed to start within {attempts * interval:.0f}s")


async def _endpoint(cluster_name: str, port: int, sky_module: Any = None) -> str:
    sky = _sky(sky_module)
    lookup = getattr(getattr(sky, "core", None), "endpoints", None) or sky.endpoints
    eps = await to_thread_typed(lambda: lookup(cluster_name, port))
    url = eps.get(port, eps.get(str(port))) if isinstance(eps, dict) else eps
    if not url:
        raise ValueError(f"cluster {cluster_name} exposes no endpoint for port {port}")
    return url if str(url).startswith("http") else f"http://{url}"


async def get_art_server_base_url(cluster_name: str, sky_module: Any = None) -> str:
    return await _endpoint(cluster_name, BACKEND_PORT, sky_module)


async def get_inference_base_url(cluster_name: str, sky_module: Any = None, port: int = INFERENCE_PORT) -> str:
    return f"{await _endpoint(cluster_name, port, sky_module)}/v1"


get_vllm_base_url = get_inference_base_url    # the reference's name for the completion-server endpoint


async def wait_for_healthcheck(base_url: str, *, attempts: int = 12, interval: float = 5.0,
                               get: Callable[[str], Awaitable[int]] | None = None) -> None:
    """Poll ``{base_url}/healthcheck`` until it answers 200; ``get`` (url -> status code) can replace httpx."""
    async def http_get(url: str) -> int:
        async with httpx.AsyncClient(timeout=10) as client:
            return (await client.get(url)).status_code

    fetch = get or http_get
    for _ in range(attempts):
        try:
            if await fetch(f"{base_url}/healthcheck") == 200:
                return
        except Exception:  # noqa: BLE001 - connection refused / reset while the server boots
            pass
        await asyncio.sleep(interval)
    raise TimeoutError(f"backend server at {base_url} did not answer /healthcheck")


async def wait_for_art_server_to_start(cluster_name: str, sky_module: Any = None, *, attempts: int = 12,
                                       interval: float = 5.0, get: Callable[[str], Awaitable[int]] | None = None) -> str:
    """Wait for the server task to run, then for its health check; returns the server's base URL."""
    await wait_for_task_to_start(cluster_name, SERVER_TASK, sky_module, attempts=attempts, interval=interval)
    base_url = await get_art_server_base_url(cluster_name, sky_module)
    await wait_for_healthcheck(base_url, attempts=attempts, interval=interval, get=get)
    return base_url
