"""Pipelined rollout batches (parity: reference ``src/art/batches.py:9-45``)."""
from __future__ import annotations

import asyncio
from typing import AsyncIterator, Awaitable, Iterable

from tqdm import auto as tqdm

from .gather import GatherContext, set_gather_context, wrap_group_awaitable
from .trajectories import TrajectoryGroup


async def trajectory_group_batches(
    groups: Iterable[Awaitable[TrajectoryGroup]],
    *,
    batch_size: int,
    max_batch_exceptions: int | float = 0,
    max_concurrent_batches: int = 4,
    skip_batches: int = 0,
    pbar_desc: str | None = "batches",
    pbar_total_completion_tokens: bool = True,
) -> AsyncIterator[list[TrajectoryGroup]]:
    """Yield lists of ``batch_size`` finished groups while later groups keep rolling out.

    Up to ``batch_size * max_concurrent_batches`` group awaitables are in flight, so a
    training step on one batch overlaps rollouts for the following ones.
    """
    waiting = list(groups)[batch_size * skip_batches:]
    running: set[asyncio.Task] = set()
    ready: list[TrajectoryGroup] = []
    ctx = GatherContext(pbar_total_completion_tokens=pbar_total_completion_tokens,
                        max_exceptions=max_batch_exceptions, increment_pbar=False)
    with set_gather_context(ctx):
        while waiting or running:
            if ctx.pbar is None:
                ctx.pbar = tqdm.tqdm(desc=pbar_desc, total=batch_size)
            while waiting and len(running) < batch_size * max_concurrent_batches:
                running.add(asyncio.create_task(wrap_group_awaitable(waiting.pop(0))))
            finished, running = await asyncio.wait(running, return_when=asyncio.FIRST_COMPLETED)
            ctx.pbar.update(len(finished))
            for task in finished:
                g = task.result()
                if g is not None:
                    ready.append(g)
            if len(ready) >= batch_size:
                ctx.pbar.close()
                ctx.reset()
                ctx.pbar_total_completion_tokens = pbar_total_completion_tokens
                ctx.max_exceptions = max_batch_exceptions
                yield ready[:batch_size]
                ready = ready[batch_size:]
        if ctx.pbar is not None:
            ctx.pbar.close()
        if ready:
            yield ready
