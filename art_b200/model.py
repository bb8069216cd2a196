"""``Model`` and ``TrainableModel`` (parity: reference ``src/art/model.py:19-344``)."""
from __future__ import annotations

from typing import TYPE_CHECKING, Any, Generic, Iterable, Optional, TypeVar

import httpx
from openai import AsyncOpenAI, DefaultAsyncHttpxClient
from pydantic import BaseModel

from . import dev
from .openai import patch_openai
from .trajectories import Trajectory, TrajectoryGroup
from .types import TrainConfig

if TYPE_CHECKING:
    from .backend import Backend

ModelConfig = TypeVar("ModelConfig", bound=BaseModel | None)


class Model(BaseModel, Generic[ModelConfig]):
    """A named policy that rollouts can query and whose results can be logged.

    A prompted (non-trainable) model carries its own ``inference_api_key`` /
    ``inference_base_url`` (and optionally ``inference_model_name``).  For a
    :class:`TrainableModel` these are filled in by ``register``.
    """

    name: str
    project: str
    config: ModelConfig | None = None
    inference_api_key: str | None = None
    inference_base_url: str | None = None
    inference_model_name: str | None = None

    _backend: Optional["Backend"] = None
    _s3_bucket: str | None = None
    _s3_prefix: str | None = None
    _openai_client: AsyncOpenAI | None = None

    @property
    def trainable(self) -> bool:
        return False

    def backend(self) -> "Backend":
        if self._backend is None:
            raise ValueError("Model is not registered with the Backend. You must call `model.register()` first.")
        return self._backend

    async def register(self, backend: "Backend") -> None:
        if self.config is not None:
            try:
                self.config.model_dump_json()
            except Exception as e:
                raise ValueError("The model config cannot be serialized to JSON. Please ensure that all "
                                 "fields are JSON serializable and try again.") from e
        self._backend = backend
        await backend.register(self)

    def openai_client(self) -> AsyncOpenAI:
        if self._openai_client is not None:
            return self._openai_client
        if self.inference_api_key is None or self.inference_base_url is None:
            if self.trainable:
                raise ValueError("OpenAI client not yet available on this trainable model. "
                                 "You must call `model.register()` first.")
            raise ValueError("In order to create an OpenAI client you must provide an "
                             "`inference_api_key` and `inference_base_url`.")
        client = AsyncOpenAI(
            base_url=self.inference_base_url,
            api_key=self.inference_api_key,
            http_client=DefaultAsyncHttpxClient(
                timeout=httpx.Timeout(timeout=1200, connect=5.0),
                limits=httpx.Limits(max_connections=100_000, max_keepalive_connections=100_000),
            ),
        )
        self._openai_client = patch_openai(client)
        return self._openai_client

    def get_inference_name(self) -> str:
        """Name to send to the inference endpoint: ``inference_model_name`` if set, else ``name``."""
        return self.inference_model_name or self.name

    async def log(self, trajectories: Iterable[Trajectory | BaseException] | Iterable[TrajectoryGroup],
                  split: str = "val") -> None:
        """Log an evaluation batch (bare trajectories are wrapped into one group)."""
        items = list(trajectories)
        if any(isinstance(t, (Trajectory, BaseException)) for t in items):
            groups = [TrajectoryGroup(items)]
        else:
            groups = items  # type: ignore[assignment]
        await self.backend()._log(self, groups, split)


class TrainableModel(Model[ModelConfig], Generic[ModelConfig]):
    base_model: str
    # Unstable: see ``dev.InternalModelConfig``.
    _internal_config: dev.InternalModelConfig | None = None

    def __init__(self, *, _internal_config: dev.InternalModelConfig | None = None, **data: Any) -> None:
        super().__init__(**data)
        if _internal_config is not None:
            object.__setattr__(self, "_internal_config", _internal_config)

    def model_dump(self, *args: Any, **kwargs: Any) -> dict:
        data = super().model_dump(*args, **kwargs)
        data["_internal_config"] = self._internal_config
        return data

    @property
    def trainable(self) -> bool:
        return True

    async def register(self, backend: "Backend", _openai_client_config: dev.OpenAIServerConfig | None = None) -> None:
        await super().register(backend)
        base_url, api_key = await backend._prepare_backend_for_training(self, _openai_client_config)
        self.inference_base_url = base_url
        self.inference_api_key = api_key
        self.inference_model_name = self.name

    async def get_step(self) -> int:
        """The model's current training step (number of completed ``train`` calls)."""
        return await self.backend()._get_step(self)

    async def delete_checkpoints(self, best_checkpoint_metric: str = "val/reward") -> None:
        """Delete all checkpoints except the latest and the best by ``best_checkpoint_metric``."""
        await self.backend()._delete_checkpoints(self, best_checkpoint_metric, benchmark_smoothing=1.0)

    async def train(self, trajectory_groups: Iterable[TrajectoryGroup], config: TrainConfig = TrainConfig(),
                    _config: dev.TrainConfig | None = None, verbose: bool = False) -> None:
        """Run one reinforcement step (GRPO) on a batch of trajectory groups."""
        async for _ in self.backend()._train_model(self, list(trajectory_groups), config, _config or {}, verbose):
            pass
