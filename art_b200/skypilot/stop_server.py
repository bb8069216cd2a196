"""``stop-server --cluster NAME``: shut down the backend server that runs on a SkyPilot cluster.

Parity: reference ``src/art/skypilot/stop_server.py:20-40`` (console script ``stop-server``,
``pyproject.toml:42``): the cluster must be UP and the server task alive; the server is asked to
close its models over HTTP, then the task is cancelled.  The cluster itself keeps running
(``SkyPilotBackend.down()`` tears it down).
"""
from __future__ import annotations

import argparse
import asyncio
from typing import Any

from .utils import SERVER_TASK, _sky, _state_name, get_art_server_base_url, is_task_created, to_thread_typed


async def stop_server(cluster_name: str, sky_module: Any = None, close_backend: bool = True) -> None:
    sky = _sky(sky_module)
    status = await to_thread_typed(lambda: sky.status(cluster_names=[cluster_name]))
    if not status or _state_name(status[0]["status"]) != "UP":
        raise ValueError(f"Cluster {cluster_name} is not running")
    if not await is_task_created(cluster_name, SERVER_TASK, sky):
        raise ValueError(f"Art server task for cluster {cluster_name} is not running")
    if close_backend:
        from ..backend import Backend

        backend = Backend(base_url=await get_art_server_base_url(cluster_name, sky))
        try:
            await backend.close()
        except Exception as e:  # noqa: BLE001 - the task is cancelled below either way
            print(f"stop-server: closing the backend over HTTP failed ({type(e).__name__}: {e}); cancelling the task")
    await to_thread_typed(lambda: sky.cancel(cluster_name=cluster_name, all=True))


def main(argv: list[str] | None = None) -> None:
    parser = argparse.ArgumentParser(description="Close the art server hosted on a skypilot cluster")
    parser.add_argument("--cluster", type=str, required=True, help="name of the skypilot cluster whose server to stop")
    args = parser.parse_args(argv)
    asyncio.run(stop_server(args.cluster))


if __name__ == "__main__":
    main()
