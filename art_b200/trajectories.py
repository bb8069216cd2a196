"""Trajectory and TrajectoryGroup (parity: reference ``src/art/trajectories.py:22-223``).

``TrajectoryGroup(...)`` accepts either finished trajectories (and exceptions), giving a
plain pydantic model, or awaitables, giving an awaitable that resolves to the group while
feeding the ambient gather context (progress bar, metric sums, exception budget).  The two
cases are separated by a metaclass ``__call__`` so that the pydantic model itself keeps an
ordinary constructor that FastAPI / ``model_validate`` can use.
"""
from __future__ import annotations

import asyncio
import time
import traceback as _tb
from contextlib import asynccontextmanager
from datetime import datetime
from typing import Any, AsyncIterator, Awaitable, Iterable, Iterator

import pydantic
from openai.types.chat.chat_completion import Choice
from pydantic._internal._model_construction import ModelMetaclass

from .types import Messages, MessagesAndChoices, Tools

MetadataValue = float | int | str | bool | None


class PydanticException(pydantic.BaseModel):
    """A serialisable record of an exception raised inside a rollout."""

    type: str
    message: str
    traceback: str

    @classmethod
    def from_exception(cls, exc: BaseException) -> "PydanticException":
        return cls(
            type=str(type(exc)),
            message=str(exc),
            traceback="\n".join(_tb.format_exception(type(exc), exc, exc.__traceback__)),
        )


class Trajectory(pydantic.BaseModel):
    messages_and_choices: MessagesAndChoices
    tools: Tools | None = None
    reward: float
    metrics: dict[str, float | int | bool] = {}
    metadata: dict[str, MetadataValue] = {}
    logs: list[str] = []
    start_time: datetime = pydantic.Field(default_factory=datetime.now, exclude=True)

    def finish(self) -> "Trajectory":
        """Record the wall-clock time since construction as ``metrics['duration']``."""
        self.metrics["duration"] = (datetime.now() - self.start_time).total_seconds()
        return self

    @asynccontextmanager
    async def track_duration(self, metric_name: str) -> AsyncIterator[None]:
        """Accumulate the time spent inside the block into ``metrics[f'{metric_name}_duration']``."""
        t0 = time.monotonic()
        try:
            yield
        finally:
            key = f"{metric_name}_duration"
            self.metrics[key] = self.metrics.get(key, 0.0) + (time.monotonic() - t0)

    def __str__(self) -> str:
        return f"Trajectory(reward={self.reward}, metrics={self.metrics}, metadata={self.metadata})"

    def messages(self) -> Messages:
        """Flatten into plain chat messages; sampled ``Choice`` objects become assistant dicts."""
        out: Messages = []
        for item in self.messages_and_choices:
            if isinstance(item, Choice):
                msg: dict[str, Any] = {"role": "assistant", "content": item.message.content}
                if item.message.tool_calls:
                    msg["tool_calls"] = [
                        {
                            "id": tc.id,
                            "type": tc.type,
                            "function": {"name": tc.function.name, "arguments": tc.function.arguments},
                        }
                        for tc in item.message.tool_calls
                    ]
                out.append(msg)  # type: ignore[arg-type]
            else:
                out.append(item)
        return out

    def for_logging(self) -> dict[str, Any]:
        rows = []
        for item in self.messages_and_choices:
            trainable = isinstance(item, Choice)
            body = item.message.to_dict() if trainable else item
            rows.append({**body, "trainable": trainable})
        return {
            "reward": self.reward,
            "metrics": self.metrics,
            "metadata": self.metadata,
            "messages": rows,
            "tools": self.tools,
            "logs": self.logs,
        }


class _PendingGroup:
    """Awaitable returned by ``TrajectoryGroup(<awaitables>)``."""

    def __init__(self, awaitables: list[Awaitable[Trajectory]], metadata: dict, exceptions: list[BaseException]):
        self._awaitables = awaitables
        self._metadata = metadata
        self._exceptions = list(exceptions)
        self._num_trajectories = len(awaitables)

    async def _run(self) -> "TrajectoryGroup":
        from .gather import get_gather_context, record_metrics

        ctx = get_gather_context()
        done: list[Trajectory] = []
        for fut in asyncio.as_completed(self._awaitables):
            try:
                traj = await fut
            except BaseException as exc:  # noqa: BLE001 - budgeted below
                self._exceptions.append(exc)
                ctx.metric_sums["exceptions"] += 1
                ctx.update_pbar(n=0)
                if ctx.too_many_exceptions():
                    raise
                continue
            done.append(traj)
            record_metrics(ctx, traj)
            ctx.update_pbar(n=1)
        return TrajectoryGroup(done, metadata=self._metadata, exceptions=self._exceptions)

    def __await__(self):
        return self._run().__await__()


class _GroupMeta(ModelMetaclass):
    def __call__(cls, trajectories: Iterable[Any] | None = None, *, metadata: dict | None = None,
                 exceptions: list | None = None, **kw: Any):
        if trajectories is None:
            trajectories = kw.pop("trajectories", [])
        items = list(trajectories)
        metadata = dict(metadata or {})
        exceptions = list(exceptions or [])
        if any(hasattr(t, "__await__") for t in items):
            return _PendingGroup(items, metadata, exceptions)
        trajs, excs = [], []
        for t in items:
            if isinstance(t, Trajectory):
                trajs.append(t)
            elif isinstance(t, BaseException):
                excs.append(t)
            elif isinstance(t, dict):
                trajs.append(Trajectory.model_validate(t))
        for e in excs + exceptions:
            pass
        records = [e if isinstance(e, PydanticException) else
                   (PydanticException.model_validate(e) if isinstance(e, dict) else PydanticException.from_exception(e))
                   for e in excs + exceptions]
        return super().__call__(trajectories=trajs, metadata=metadata, exceptions=records)


class TrajectoryGroup(pydantic.BaseModel, metaclass=_GroupMeta):
    trajectories: list[Trajectory]
    metadata: dict[str, MetadataValue] = {}
    exceptions: list[PydanticException] = []

    def __iter__(self) -> Iterator[Trajectory]:  # type: ignore[override]
        return iter(self.trajectories)

    def __len__(self) -> int:
        return len(self.trajectories)
