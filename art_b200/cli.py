"""``python -m art_b200.cli run [--host H] [--port 7999]``: serve a LocalBackend over HTTP.

Routes and payloads are the ones :class:`art_b200.backend.Backend` speaks (parity: reference
``src/art/cli.py:17-140``): one POST per backend method, ``/_train_model`` answers with one JSON
line per optimizer step.  ``build_app`` is separate from ``run`` so tests can mount the app on
an in-process ASGI transport with any backend object.
"""
from __future__ import annotations

import json
import socket
from typing import Any, AsyncIterator

import typer
from fastapi import Body, FastAPI
from fastapi.responses import StreamingResponse

from . import dev
from .model import Model, TrainableModel
from .trajectories import TrajectoryGroup
from .types import TrainConfig
from .utils.deploy_model import LoRADeploymentProvider

app = typer.Typer()


def _model_from(payload: dict[str, Any]) -> Model:
    """Rebuild a Model / TrainableModel (with its private internal config) from ``model_dump()``."""
    data = dict(payload)
    internal = data.pop("_internal_config", None)
    if "base_model" in data:
        return TrainableModel(**data, _internal_config=internal)
    return Model(**data)


def build_app(backend) -> FastAPI:
    api = FastAPI(title="art-b200 backend")

    @api.get("/healthcheck")
    async def healthcheck():
        return {"status": "ok"}

    @api.post("/close")
    async def close():
        r = backend.close()
        if hasattr(r, "__await__"):
            await r

    @api.post("/register")
    async def register(model: dict = Body(...)):
        await backend.register(_model_from(model))

    @api.post("/_get_step")
    async def get_step(model: dict = Body(...)):
        return await backend._get_step(_model_from(model))

    @api.post("/_delete_checkpoints")
    async def delete_checkpoints(model: dict = Body(...), benchmark: str = "val/reward", benchmark_smoothing: float = 1.0):
        await backend._delete_checkpoints(_model_from(model), benchmark, benchmark_smoothing)

    @api.post("/_prepare_backend_for_training")
    async def prepare(model: dict = Body(...), config: dict | None = Body(None)):
        base_url, api_key = await backend._prepare_backend_for_training(_model_from(model), config)
        return [base_url, api_key]

    @api.post("/_log")
    async def log(model: dict = Body(...), trajectory_groups: list[dict] = Body(...), split: str = Body("val")):
        groups = [TrajectoryGroup.model_validate(g) for g in trajectory_groups]
        await backend._log(_model_from(model), groups, split)

    @api.post("/_train_model")
    async def train_model(model: dict = Body(...), trajectory_groups: list[dict] = Body(...),
                          config: dict = Body(...), dev_config: dict = Body(default_factory=dict),
                          verbose: bool = Body(False)) -> StreamingResponse:
        groups = [TrajectoryGroup.model_validate(g) for g in trajectory_groups]
        m = _model_from(model)

        async def stream() -> AsyncIterator[str]:
            try:
                async for result in backend._train_model(m, groups, TrainConfig(**config), dev_config, verbose):
                    yield json.dumps(result) + "\n"
            except Exception as e:  # the status line is already sent: report in-band
                yield json.dumps({"error": f"{type(e).__name__}: {e}"}) + "\n"

        return StreamingResponse(stream(), media_type="application/x-ndjson")

    @api.post("/_experimental_pull_from_s3")
    async def pull(model: dict = Body(...), s3_bucket: str | None = Body(None), prefix: str | None = Body(None),
                   verbose: bool = Body(False), delete: bool = Body(False)):
        await backend._experimental_pull_from_s3(model=_model_from(model), s3_bucket=s3_bucket, prefix=prefix,
                                                 verbose=verbose, delete=delete)

    @api.post("/_experimental_push_to_s3")
    async def push(model: dict = Body(...), s3_bucket: str | None = Body(None), prefix: str | None = Body(None),
                   verbose: bool = Body(False), delete: bool = Body(False)):
        await backend._experimental_push_to_s3(model=_model_from(model), s3_bucket=s3_bucket, prefix=prefix,
                                               verbose=verbose, delete=delete)

    @api.post("/_experimental_deploy")
    async def deploy(deploy_to: LoRADeploymentProvider = Body(...), model: dict = Body(...), step: int | None = Body(None),
                     s3_bucket: str | None = Body(None), prefix: str | None = Body(None), verbose: bool = Body(False),
                     pull_s3: bool = Body(True), wait_for_completion: bool = Body(True)):
        job = await backend._experimental_deploy(deploy_to=deploy_to, model=_model_from(model), step=step,
                                                 s3_bucket=s3_bucket, prefix=prefix, verbose=verbose, pull_s3=pull_s3,
                                                 wait_for_completion=wait_for_completion)
        return job.model_dump()

    return api


@app.command()
def run(host: str = "0.0.0.0", port: int = 7999) -> None:
    """Start the backend server."""
    import uvicorn

    from .local import LocalBackend

    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        if s.connect_ex(("127.0.0.1", port)) == 0:
            print(f"Port {port} is already in use, possibly because the server is already running.")
            return
    uvicorn.run(build_app(LocalBackend()), host=host, port=port, loop="asyncio")


@app.command()
def version() -> None:
    from . import __version__

    print(__version__)


if __name__ == "__main__":
    app()
