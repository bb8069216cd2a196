"""Run an object in a spawned child process behind a transparent proxy.

``proxy = move_to_child_process(service, log_file=..., process_name=...)`` pickles ``service``
into a ``spawn``-started child; attribute access on the proxy returns callables that forward
to the child.  Plain methods and coroutine methods return an awaitable; async-generator
methods return an async iterator whose items stream back one by one (this is how training
metrics reach the backend while a train call is still running).  Exceptions raised in the
child are re-raised in the parent with the child's formatted traceback attached as
``__remote_traceback__`` and appended to the message.

Behavioural parity: reference ``src/mp_actors/move.py:27-247`` and ``traceback.py:11-52``.
Differences: no dependency on ``tblib`` (the traceback travels as text), one reader thread
instead of an executor per call, and ``close()`` is idempotent and joins with a deadline
before escalating terminate -> kill.
"""
from __future__ import annotations

import asyncio
import inspect
import itertools
import multiprocessing as mp
import os
import pickle
import sys
import threading
import traceback
from dataclasses import dataclass
from typing import Any, TypeVar

T = TypeVar("T")
_ctx = mp.get_context("spawn")
_SHUTDOWN = "__shutdown__"


class ActorDiedError(RuntimeError):
    """The child process behind a proxy exited while (or before) a call was in flight."""


class RemoteError(RuntimeError):
    """Raised in the parent when the child's exception cannot be unpickled."""


@dataclass
class _Request:
    id: int
    method: str
    args: tuple
    kwargs: dict
    kind: str = "call"     # call | next | aclose


@dataclass
class _Response:
    id: int
    kind: str              # result | error | item | stop
    payload: Any = None
    tb: str | None = None


def move_to_child_process(obj: T, log_file: str | None = None, process_name: str | None = None) -> T:
    return Proxy(obj, log_file, process_name)  # type: ignore[return-value]


class Proxy:
    def __init__(self, obj: object, log_file: str | None = None, process_name: str | None = None):
        self._cls = type(obj)
        self._requests = _ctx.Queue()
        self._responses = _ctx.Queue()
        self._process = _ctx.Process(target=_child_main, name=process_name or "art-b200-actor",
                                     args=(obj, self._requests, self._responses, log_file, process_name), daemon=True)
        self._process.start()
        self._ids = itertools.count(1)
        self._pending: dict[int, tuple[asyncio.AbstractEventLoop, asyncio.Future]] = {}
        self._streams: dict[int, tuple[asyncio.AbstractEventLoop, asyncio.Queue]] = {}
        self._lock = threading.Lock()
        self._closed = False
        self._reader = threading.Thread(target=self._read_loop, daemon=True)
        self._reader.start()

    # -- plumbing ---------------------------------------------------------------------------
    def _read_loop(self) -> None:
        while True:
            try:
                resp: _Response = self._responses.get()
            except (EOFError, OSError):
                return
            if resp.id == 0 and resp.kind == "stop":
                return
            with self._lock:
                stream = self._streams.get(resp.id)
                pending = self._pending.pop(resp.id, None) if stream is None else None
            if stream is not None:
                loop, q = stream
                loop.call_soon_threadsafe(q.put_nowait, resp)
            elif pending is not None:
                loop, fut = pending
                loop.call_soon_threadsafe(_resolve, fut, resp)

    def _submit(self, req: _Request) -> asyncio.Future:
        if self._closed:
            raise RuntimeError("actor is closed")
        if not self._process.is_alive():
            raise ActorDiedError(f"actor process died (exit code {self._process.exitcode})")
        loop = asyncio.get_running_loop()
        fut = loop.create_future()
        with self._lock:
            self._pending[req.id] = (loop, fut)
        self._requests.put(req)
        return fut

    def __getattr__(self, name: str):
        if name.startswith("_"):
            raise AttributeError(name)
        attr = getattr(self._cls, name, None)
        if attr is not None and inspect.isasyncgenfunction(attr):
            def start(*args: Any, **kwargs: Any):
                return self._stream(name, args, kwargs)
            return start

        async def call(*args: Any, **kwargs: Any):
            return await self._await_reply(self._submit(_Request(next(self._ids), name, args, kwargs)))
        return call

    async def _await_reply(self, fut: asyncio.Future):
        """Wait for the child's answer, failing the call if the child process disappears."""
        while True:
            done, _ = await asyncio.wait({fut}, timeout=1.0)
            if done:
                return fut.result()
            if not self._process.is_alive():
                fut.cancel()
                raise ActorDiedError(f"actor process died (exit code {self._process.exitcode})")

    async def _stream(self, name: str, args: tuple, kwargs: dict):
        rid = next(self._ids)
        loop = asyncio.get_running_loop()
        q: asyncio.Queue = asyncio.Queue()
        with self._lock:
            self._streams[rid] = (loop, q)
        self._requests.put(_Request(rid, name, args, kwargs, kind="call"))
        try:
            while True:
                resp = await self._next_or_death(q)
                if resp.kind == "item":
                    yield resp.payload
                    self._requests.put(_Request(rid, name, (), {}, kind="next"))
                elif resp.kind == "stop":
                    return
                else:
                    raise _rebuild(resp)
        finally:
            with self._lock:
                self._streams.pop(rid, None)
            if not self._closed and self._process.is_alive():
                self._requests.put(_Request(rid, name, (), {}, kind="aclose"))

    async def _next_or_death(self, q: asyncio.Queue) -> _Response:
        while True:
            try:
                return await asyncio.wait_for(q.get(), timeout=1.0)
            except asyncio.TimeoutError:
                if not self._process.is_alive():
                    raise ActorDiedError(f"actor process died (exit code {self._process.exitcode})") from None

    def close(self, timeout: float = 5.0) -> None:
        if self._closed:
            return
        self._closed = True
        try:
            self._requests.put(_Request(0, _SHUTDOWN, (), {}))
        except Exception:
            pass
        self._process.join(timeout)
        if self._process.is_alive():
            self._process.terminate()
            self._process.join(2.0)
        if self._process.is_alive():
            self._process.kill()
            self._process.join(2.0)
        try:
            self._responses.put(_Response(0, "stop"))
        except Exception:
            pass
        with self._lock:
            pend, self._pending = self._pending, {}
        for loop, fut in pend.values():
            try:
                loop.call_soon_threadsafe(_cancel, fut)
            except RuntimeError:  # that loop is already closed
                pass

    def __del__(self):
        try:
            self.close(timeout=0.5)
        except Exception:
            pass


def _cancel(fut: asyncio.Future) -> None:
    if not fut.done():
        fut.set_exception(RuntimeError("actor closed"))


def _rebuild(resp: _Response) -> BaseException:
    exc = resp.payload
    if not isinstance(exc, BaseException):
        exc = RemoteError(str(exc))
    exc.__remote_traceback__ = resp.tb  # type: ignore[attr-defined]
    if resp.tb:
        try:
            exc.add_note("--- traceback in the actor process ---\n" + resp.tb)
        except Exception:
            pass
    return exc


def _resolve(fut: asyncio.Future, resp: _Response) -> None:
    if fut.done():
        return
    if resp.kind == "result":
        fut.set_result(resp.payload)
    else:
        fut.set_exception(_rebuild(resp))


# ------------------------------------------------------------------------------ child side
def _safe_exc(e: BaseException) -> Any:
    try:
        pickle.loads(pickle.dumps(e))
        return e
    except Exception:
        return RemoteError(f"{type(e).__name__}: {e}")


def _child_main(obj: object, requests, responses, log_file: str | None, process_name: str | None) -> None:
    if process_name:
        try:
            import setproctitle

            setproctitle.setproctitle(process_name)
        except Exception:
            pass
    if log_file:
        os.makedirs(os.path.dirname(log_file) or ".", exist_ok=True)
        f = open(log_file, "a", buffering=1)
        sys.stdout = sys.stderr = f
    asyncio.run(_serve(obj, requests, responses))


async def _serve(obj: object, requests, responses) -> None:
    loop = asyncio.get_running_loop()
    gens: dict[int, Any] = {}
    tasks: set[asyncio.Task] = set()

    def send(resp: _Response) -> None:
        try:
            responses.put(resp)
        except Exception:
            responses.put(_Response(resp.id, "error", RemoteError(f"unpicklable result: {type(resp.payload).__name__}"), None))

    async def advance(rid: int) -> None:
        gen = gens.get(rid)
        if gen is None:
            return
        try:
            item = await gen.__anext__()
            send(_Response(rid, "item", item))
        except StopAsyncIteration:
            gens.pop(rid, None)
            send(_Response(rid, "stop"))
        except BaseException as e:  # noqa: BLE001
            gens.pop(rid, None)
            send(_Response(rid, "error", _safe_exc(e), traceback.format_exc()))

    async def handle(req: _Request) -> None:
        try:
            if req.kind == "next":
                await advance(req.id)
                return
            if req.kind == "aclose":
                gen = gens.pop(req.id, None)
                if gen is not None:
                    await gen.aclose()
                return
            attr = getattr(obj, req.method)
            if inspect.isasyncgenfunction(attr):
                gens[req.id] = attr(*req.args, **req.kwargs)
                await advance(req.id)
                return
            result = attr(*req.args, **req.kwargs) if callable(attr) else attr
            if inspect.isawaitable(result):
                result = await result
            send(_Response(req.id, "result", result))
        except BaseException as e:  # noqa: BLE001
            send(_Response(req.id, "error", _safe_exc(e), traceback.format_exc()))

    while True:
        req: _Request = await loop.run_in_executor(None, requests.get)
        if req.method == _SHUTDOWN:
            break
        t = asyncio.create_task(handle(req))
        tasks.add(t)
        t.add_done_callback(tasks.discard)
    for t in list(tasks):
        t.cancel()
    closer = getattr(obj, "shutdown", None)
    if callable(closer):
        try:
            r = closer()
            if inspect.isawaitable(r):
                await r
        except Exception:
            pass


def streamline_tracebacks(exc: BaseException) -> BaseException:
    """Drop this module's frames from ``exc.__traceback__`` so user code sees its own call site."""
    tb = exc.__traceback__
    keep = []
    while tb is not None:
        if tb.tb_frame.f_code.co_filename != __file__:
            keep.append(tb)
        tb = tb.tb_next
    new = None
    for t in reversed(keep):
        import types

        new = types.TracebackType(new, t.tb_frame, t.tb_lasti, t.tb_lineno)
    return exc.with_traceback(new)
