"""Concurrent rollout gathering with live metrics (parity: reference ``src/art/gather.py:13-230``)."""
from __future__ import annotations

import asyncio
import contextlib
import contextvars
from collections import Counter
from dataclasses import dataclass, field
from typing import Awaitable, Iterable, Iterator

from openai.types.chat.chat_completion import Choice
from tqdm import auto as tqdm

from .trajectories import Trajectory, TrajectoryGroup

_TOKEN_KEYS = ("prompt_tokens", "completion_tokens", "total_completion_tokens")


@dataclass
class GatherContext:
    """Ambient state shared by every rollout inside one ``gather_*`` call."""

    pbar: "tqdm.tqdm | None" = None
    metric_sums: Counter = field(default_factory=Counter)
    metric_divisors: Counter = field(default_factory=Counter)
    max_metrics: int | None = None
    pbar_total_completion_tokens: bool = False
    max_exceptions: int | float = 0
    increment_pbar: bool = True

    def update_pbar(self, n: int) -> None:
        if self.pbar is None:
            return
        if self.increment_pbar:
            self.pbar.update(n)
        names = list(self.metric_sums)
        if self.max_metrics is not None:
            names = names[: self.max_metrics]
        shown = {k: self.metric_sums[k] / max(1, self.metric_divisors[k]) for k in names}
        for k in _TOKEN_KEYS:  # token counters go last
            if k in shown:
                shown[k] = shown.pop(k)
        self.pbar.set_postfix(shown)

    def too_many_exceptions(self) -> bool:
        """Budget is an absolute count, or a fraction of the bar total when in (0, 1)."""
        n = self.metric_sums["exceptions"]
        if 0 < self.max_exceptions < 1 and self.pbar is not None and self.pbar.total:
            if n / self.pbar.total <= self.max_exceptions:
                return False
        return n > self.max_exceptions

    def reset(self) -> None:
        self.pbar = None
        self.metric_sums = Counter()
        self.metric_divisors = Counter()
        self.pbar_total_completion_tokens = False
        self.max_exceptions = 0


_ctx_var: contextvars.ContextVar[GatherContext] = contextvars.ContextVar("art_b200_gather", default=GatherContext())


@contextlib.contextmanager
def set_gather_context(context: GatherContext) -> Iterator[None]:
    tok = _ctx_var.set(context)
    try:
        yield
    finally:
        _ctx_var.reset(tok)


def get_gather_context() -> GatherContext:
    return _ctx_var.get()


def record_metrics(context: GatherContext, trajectory: Trajectory) -> None:
    lps = [m.logprobs for m in trajectory.messages_and_choices if isinstance(m, Choice) and m.logprobs]
    if lps:
        trajectory.metrics["completion_tokens"] = sum(len(l.content or l.refusal or []) for l in lps) / len(lps)
    context.metric_sums["reward"] += trajectory.reward  # type: ignore[assignment]
    context.metric_divisors["reward"] += 1
    context.metric_sums.update(trajectory.metrics)
    context.metric_divisors.update(trajectory.metrics.keys())


async def wrap_group_awaitable(awaitable: Awaitable[TrajectoryGroup]) -> TrajectoryGroup | None:
    if hasattr(awaitable, "_num_trajectories"):
        return await awaitable  # accounts for itself
    ctx = get_gather_context()
    try:
        group = await awaitable
    except BaseException:
        ctx.metric_sums["exceptions"] += 1
        ctx.update_pbar(n=0)
        if ctx.too_many_exceptions():
            raise
        return None
    for t in group:
        record_metrics(ctx, t)
    ctx.update_pbar(n=len(group))
    return group


async def wrap_trajectories_awaitable(awaitable):
    ctx = get_gather_context()
    try:
        result = await awaitable
    except BaseException as exc:
        ctx.metric_sums["exceptions"] += 1
        ctx.update_pbar(n=0)
        if ctx.too_many_exceptions():
            raise
        return exc
    if isinstance(result, Trajectory):
        record_metrics(ctx, result)
        ctx.update_pbar(n=1)
        return result
    result = list(result)
    for t in result:
        record_metrics(ctx, t)
    ctx.update_pbar(n=1)
    return result


async def gather_trajectory_groups(
    groups: Iterable[Awaitable[TrajectoryGroup]],
    *,
    pbar_desc: str | None = "gather",
    pbar_total_completion_tokens: bool = True,
    max_exceptions: int | float = 0,
    max_metrics: int | None = None,
) -> list[TrajectoryGroup]:
    groups = list(groups)
    ctx = GatherContext(pbar_total_completion_tokens=pbar_total_completion_tokens,
                        max_exceptions=max_exceptions, max_metrics=max_metrics)
    with set_gather_context(ctx):
        fut = asyncio.gather(*[wrap_group_awaitable(g) for g in groups])
        ctx.pbar = tqdm.tqdm(desc=pbar_desc, total=sum(getattr(g, "_num_trajectories", 1) for g in groups))
        try:
            results = await fut
        finally:
            ctx.pbar.close()
    return [g for g in results if g is not None]


async def gather_trajectories(
    trajectories: Iterable[Awaitable],
    *,
    pbar_desc: str | None = "gather",
    pbar_total_completion_tokens: bool = True,
    max_exceptions: int | float = 0,
) -> list:
    """Await trajectories (or iterables of trajectories); failures within budget are returned in place."""
    items = list(trajectories)
    ctx = GatherContext(pbar=tqdm.tqdm(desc=pbar_desc, total=len(items)),
                        pbar_total_completion_tokens=pbar_total_completion_tokens, max_exceptions=max_exceptions)
    with set_gather_context(ctx):
        try:
            results = await asyncio.gather(*[wrap_trajectories_awaitable(t) for t in items])
        finally:
            if ctx.pbar is not None:
                ctx.pbar.close()
    return list(results)
