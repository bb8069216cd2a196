"""Turn ``httpx.HTTPStatusError`` into an exception that shows the server's ``detail``
(parity: reference ``src/art/utils/log_http_errors.py:5-21``)."""
import functools

import httpx


def log_http_errors(func):
    @functools.wraps(func)
    async def wrapper(*a, **kw):
        try:
            return await func(*a, **kw)
        except httpx.HTTPStatusError as e:
            try:
                detail = e.response.json().get("detail")
            except Exception:
                raise e
            raise Exception(f"[HTTP {e.response.status_code}] {e.request.url} {detail}") from e
    return wrapper
