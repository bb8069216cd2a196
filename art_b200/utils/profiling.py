"""Tracing and phase timing.

* :func:`nvtx_range` - NVTX range (shows up in Nsight timelines) around a phase; a no-op without CUDA.
* :class:`PhaseTimer` - per-phase CUDA-event timing of a step (``with timer.phase("backward"): ...``); the summary is
  milliseconds per phase, optionally the maximum over the ranks of a process group, and can be appended to a JSON-lines
  file.  On CPU it falls back to ``time.perf_counter``.
* :class:`ChromeTrace` - host-side event recorder for the rollout scheduler (one "X" event per engine step, counters
  for running / waiting sequences and free KV blocks); ``save`` writes the Chrome ``chrome://tracing`` / Perfetto JSON.

The reference has no profiler integration of its own (``src/art/dev/engine.py:77,105-106`` only forwards tracing knobs
to the inference library); rollout timing there is ``Trajectory.track_duration`` (``src/art/trajectories.py:35-48``).
Enable from the environment: ``ARTB_PHASE_TIMING=1`` (trainer) and ``ARTB_TRACE_FILE=/path/trace.json`` (engine).
"""
from __future__ import annotations

import contextlib
import json
import os
import threading
import time
from collections import defaultdict

import torch


@contextlib.contextmanager
def nvtx_range(name: str):
    if torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


class PhaseTimer:
    def __init__(self, device: torch.device | str | None = None, enabled: bool = True):
        self.device = torch.device(device) if device is not None else None
        self.cuda = self.device is not None and self.device.type == "cuda"
        self.enabled = enabled
        self._pending: list[tuple[str, object, object]] = []
        self.totals: dict[str, float] = defaultdict(float)
        self.counts: dict[str, int] = defaultdict(int)

    @contextlib.contextmanager
    def phase(self, name: str):
        if not self.enabled:
            yield
            return
        with nvtx_range(name):
            if self.cuda:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                try:
                    yield
                finally:
                    e1.record()
                    self._pending.append((name, e0, e1))
            else:
                t0 = time.perf_counter()
                try:
                    yield
                finally:
                    self.totals[name] += (time.perf_counter() - t0) * 1e3
                    self.counts[name] += 1

    def _flush(self) -> None:
        if self._pending:
            torch.cuda.synchronize(self.device)
            for name, e0, e1 in self._pending:
                self.totals[name] += e0.elapsed_time(e1)
                self.counts[name] += 1
            self._pending.clear()

    def summary(self, group=None, reset: bool = True) -> dict[str, float]:
        """Milliseconds per phase since the last reset; with ``group`` the maximum over its ranks."""
        self._flush()
        out = {k: round(v, 4) for k, v in self.totals.items()}
        if group is not None and out:
            import torch.distributed as dist

            keys = sorted(out)
            t = torch.tensor([out[k] for k in keys], dtype=torch.float64,
                             device=self.device if self.cuda else "cpu")
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
            out = {k: round(float(v), 4) for k, v in zip(keys, t.tolist())}
        if reset:
            self.totals.clear()
            self.counts.clear()
        return out

    def dump_jsonl(self, path: str, extra: dict | None = None, group=None) -> dict:
        rec = {"phases_ms": self.summary(group), **(extra or {})}
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        with open(path, "a") as f:
            f.write(json.dumps(rec) + "\n")
        return rec


class ChromeTrace:
    """Minimal Chrome trace-event writer (thread-safe)."""

    def __init__(self, process_name: str = "art_b200"):
        self._events: list[dict] = [{"name": "process_name", "ph": "M", "pid": os.getpid(), "args": {"name": process_name}}]
        self._lock = threading.Lock()
        self._t0 = time.perf_counter()

    def _ts(self) -> float:
        return (time.perf_counter() - self._t0) * 1e6

    @contextlib.contextmanager
    def span(self, name: str, cat: str = "host", **args):
        t0 = self._ts()
        try:
            yield
        finally:
            with self._lock:
                self._events.append({"name": name, "cat": cat, "ph": "X", "ts": t0, "dur": self._ts() - t0,
                                     "pid": os.getpid(), "tid": threading.get_ident() % 100000, "args": args})

    def counter(self, name: str, **values) -> None:
        with self._lock:
            self._events.append({"name": name, "ph": "C", "ts": self._ts(), "pid": os.getpid(), "args": values})

    def instant(self, name: str, **args) -> None:
        with self._lock:
            self._events.append({"name": name, "ph": "i", "s": "p", "ts": self._ts(), "pid": os.getpid(),
                                 "tid": threading.get_ident() % 100000, "args": args})

    def save(self, path: str) -> None:
        with self._lock:
            data = {"traceEvents": list(self._events), "displayTimeUnit": "ms"}
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        with open(path, "w") as f:
            json.dump(data, f)
