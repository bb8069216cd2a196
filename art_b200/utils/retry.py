"""Retry decorator with exponential backoff for sync and async callables
(parity: reference ``src/art/utils/retry.py:19-107``)."""
from __future__ import annotations

import asyncio
import functools
import inspect
import logging
import time
from typing import Any, Callable, TypeVar

F = TypeVar("F", bound=Callable[..., Any])
log = logging.getLogger(__name__)


def retry(max_attempts: int = 3, delay: float = 0.25, backoff_factor: float = 2.0,
          exceptions: tuple[type[BaseException], ...] = (Exception,),
          on_retry: Callable[[BaseException, int], None] | None = None) -> Callable[[F], F]:
    """Re-run the wrapped callable up to ``max_attempts`` times on the listed exceptions.

    The pause before attempt *k+1* is ``delay * backoff_factor**(k-1)``.  ``on_retry(exc, attempt)``
    is invoked before each pause.  The last failure is re-raised unchanged.
    """
    if max_attempts < 1:
        raise ValueError("max_attempts must be >= 1")

    def _pause(attempt: int) -> float:
        return delay * (backoff_factor ** (attempt - 1))

    def deco(fn: F) -> F:
        if inspect.iscoroutinefunction(fn):
            @functools.wraps(fn)
            async def awrapper(*a: Any, **kw: Any):
                for attempt in range(1, max_attempts + 1):
                    try:
                        return await fn(*a, **kw)
                    except exceptions as exc:
                        if attempt == max_attempts:
                            raise
                        if on_retry:
                            on_retry(exc, attempt)
                        else:
                            log.warning("retry %d/%d of %s after %r", attempt, max_attempts, fn.__name__, exc)
                        await asyncio.sleep(_pause(attempt))
            return awrapper  # type: ignore[return-value]

        @functools.wraps(fn)
        def wrapper(*a: Any, **kw: Any):
            for attempt in range(1, max_attempts + 1):
                try:
                    return fn(*a, **kw)
                except exceptions as exc:
                    if attempt == max_attempts:
                        raise
                    if on_retry:
                        on_retry(exc, attempt)
                    else:
                        log.warning("retry %d/%d of %s after %r", attempt, max_attempts, fn.__name__, exc)
                    time.sleep(_pause(attempt))
        return wrapper  # type: ignore[return-value]

    return deco
