"""Per-key concurrency limit for coroutines
(parity: reference ``src/art/utils/limit_concurrency.py:6-25``)."""
from __future__ import annotations

import asyncio
import functools
from typing import Callable


def limit_concurrency(n: int, derive_key: Callable[..., str] | None = None):
    """At most ``n`` concurrent executions per key (one shared key when ``derive_key`` is None)."""
    gates: dict[str, asyncio.Semaphore] = {}

    def deco(fn):
        @functools.wraps(fn)
        async def wrapper(*a, **kw):
            key = derive_key(*a, **kw) if derive_key else "default"
            gate = gates.setdefault(key, asyncio.Semaphore(n))
            async with gate:
                return await fn(*a, **kw)
        return wrapper

    return deco
