"""An ASGI middleware function that tests name by import path."""


async def add_header(request, call_next):
    response = await call_next(request)
    response.headers["X-Test-Middleware"] = "1"
    return response
