"""Lockstep control of the engines of one tensor-parallel replica.

A tensor-parallel :class:`~art_b200.engine.runner.NativeRunner` issues collectives inside every
prefill and decode call, so all ranks of the replica must make the same scheduler decisions in
the same order.  ``ReplicaEngine`` guarantees that by construction: rank 0 of ``ctrl_group`` (a
CPU / gloo group over the replica's ranks) is the *leader* and owns the public API; nothing it is
told takes effect at once.  Requests, aborts, adapter loads, scoring jobs and cache operations are
queued, and at the start of every scheduler step the leader broadcasts the queued commands; every
rank applies them in the same order and then runs the same ``Engine.step()``.  Sampling seeds are
resolved by the leader and travel with the request, so every rank draws the same tokens (the
vocabulary-parallel sampler already returns identical tokens on all ranks).  Followers sit in
``follow()`` until the leader shuts down.  An idle leader sends a keep-alive tick so that followers
never run into the group's collective timeout.

Failure detection: every tick ends with a one-integer all-reduce over the control group in which a
rank that raised (a bad adapter, an allocation failure, a kernel status error) reports it.  The
failing rank re-raises its own exception, the others raise ``ReplicaError`` at the same tick, so
nobody is left waiting in a later broadcast.  (A rank that dies inside a step that contains GPU
collectives is caught by the collective library's own timeout, not here.)

The reference reaches multi-GPU serving through vLLM's own executor (src/art/dev/engine.py:
tensor_parallel_size); this is the equivalent for the native engine.
"""
from __future__ import annotations

import dataclasses
import time

import torch
import torch.distributed as dist

from .engine import Engine, SamplingParams, Sequence


class ReplicaError(RuntimeError):
    """A rank of the replica failed while applying commands or stepping; the replica must be rebuilt."""


class _NoLoop:
    """Stand-in event loop of follower ranks: results of scoring jobs are dropped there."""

    @staticmethod
    def call_soon_threadsafe(fn, *args):
        return None


class ReplicaEngine(Engine):
    def __init__(self, runner, block_manager, *, ctrl_group, keepalive_s: float = 60.0, **kw):
        super().__init__(runner, block_manager, **kw)
        self.ctrl = ctrl_group
        self.leader_rank = dist.get_global_rank(ctrl_group, 0)
        self.is_leader = dist.get_rank() == self.leader_rank
        self.keepalive_s = keepalive_s
        self._pending: list[tuple] = []          # leader: commands not yet broadcast
        self._seq_of: dict[int, Sequence] = {}   # request id -> this rank's sequence
        self._next_rid = 0
        self._last_tick = time.monotonic()
        self._applying = False                   # inside _apply: the overridden methods act locally
        self._device = getattr(runner, "device", torch.device("cpu"))

    # -- leader API ---------------------------------------------------------------------------------
    def _leader_only(self) -> None:
        if not self.is_leader:
            raise RuntimeError("only the leader rank of a replica takes requests; followers call follow()")

    def add_request(self, prompt_ids, params: SamplingParams, adapter_name=None, loop=None) -> Sequence:
        self._leader_only()
        seq = self._new_sequence(prompt_ids, params, adapter_name, loop)
        wire = dataclasses.asdict(dataclasses.replace(params, seed=seq.seed))     # the resolved seed travels
        with self._lock:
            rid = self._next_rid
            self._next_rid += 1
            self._seq_of[rid] = seq
            seq.rid = rid
            self._pending.append(("add", rid, list(prompt_ids), wire, adapter_name))
        self._wake.set()
        return seq

    def abort(self, seq: Sequence) -> None:
        self._leader_only()
        with self._lock:
            self._pending.append(("abort", seq.rid))
        self._wake.set()

    def _call_everywhere(self, method: str, *args):
        """Queue ``Engine.<method>(*args)`` for every rank and apply it now, between steps, without stepping."""
        if self._applying:                       # reached from inside an applied command (e.g. sleep -> reset cache)
            return getattr(Engine, method)(self, *args)
        self._leader_only()
        with self._lock:
            self._pending.append(("call", method, args))
        with self._step_lock:
            self._tick(step=False)

    def set_adapter(self, name: str, state: dict | None) -> int:
        if self._applying:
            return Engine.set_adapter(self, name, state)
        cpu = None if state is None else {k: v.detach().to("cpu") for k, v in state.items()}
        self._call_everywhere("set_adapter", name, cpu)
        return self.adapters[name]

    def set_vocabulary(self, vocab, eos_token_id=None) -> None:
        self._call_everywhere("set_vocabulary", vocab, eos_token_id)      # followers constrain the same way

    def remove_adapter(self, name: str) -> None:
        self._call_everywhere("remove_adapter", name)

    def reset_prefix_cache(self) -> None:
        self._call_everywhere("reset_prefix_cache")

    def sleep(self, level: int = 1) -> None:
        self._call_everywhere("sleep", level)

    def wake_up(self) -> None:
        self._call_everywhere("wake_up")

    async def score(self, prompt_ids, completion_ids, adapter_name=None):
        import asyncio

        self._leader_only()
        adapter = -1 if adapter_name is None else self.adapters[adapter_name]
        loop = asyncio.get_running_loop()
        fut = loop.create_future()
        with self._lock:
            rid = self._next_rid
            self._next_rid += 1
            self._seq_of[rid] = (loop, fut)
            self._pending.append(("score", rid, list(prompt_ids) + list(completion_ids), len(prompt_ids), adapter))
        self._wake.set()
        if self._thread is None:
            self.step()
        return await fut

    # -- the tick -----------------------------------------------------------------------------------
    def _apply(self, cmd: tuple) -> None:
        kind = cmd[0]
        if kind == "add":
            _, rid, prompt_ids, wire, adapter_name = cmd
            if self.is_leader:
                seq = self._seq_of[rid]
            else:
                seq = self._new_sequence(prompt_ids, SamplingParams(**wire), adapter_name, None)
                seq.rid = rid
                self._seq_of[rid] = seq
            with self._lock:
                self.waiting.append(seq)
        elif kind == "abort":
            seq = self._seq_of.get(cmd[1])
            if isinstance(seq, Sequence):
                seq.aborted = True
        elif kind == "score":
            _, rid, toks, n_prompt, adapter = cmd
            loop, fut = self._seq_of.pop(rid) if self.is_leader else (_NoLoop, None)
            self.score_queue.append((toks, n_prompt, adapter, loop, fut))
        elif kind == "call":
            _, method, args = cmd
            if method == "set_adapter" and args[1] is not None:
                args = (args[0], {k: v.to(self._device) for k, v in args[1].items()})
            self._applying = True
            try:
                getattr(Engine, method)(self, *args)
            finally:
                self._applying = False
        else:
            raise ValueError(f"unknown replica command {kind!r}")

    def _tick(self, step: bool, stop: bool = False) -> bool:
        """Leader: broadcast the queued commands; everyone: apply them, then (optionally) step."""
        if self.is_leader:
            with self._lock:
                cmds, self._pending = self._pending, []
            box = [{"cmds": cmds, "step": step, "stop": stop}]
        else:
            box = [None]
        dist.broadcast_object_list(box, src=self.leader_rank, group=self.ctrl)
        msg = box[0]
        self._last_tick = time.monotonic()
        worked, failure = False, None
        try:
            if self.error is not None:
                raise ReplicaError("this replica already failed") from self.error
            for cmd in msg["cmds"]:
                self._apply(cmd)
            if len(self._seq_of) > 4096:             # forget finished requests
                self._seq_of = {r: q for r, q in self._seq_of.items() if not (isinstance(q, Sequence) and q.finished)}
            if msg["stop"]:
                self._stop = True
            elif msg["step"]:
                worked = Engine.step(self)
        except BaseException as e:  # noqa: BLE001 - reported to the peers below, then re-raised
            failure = e
        flag = torch.tensor([0 if failure is None else 1], dtype=torch.int32)
        dist.all_reduce(flag, group=self.ctrl)
        if failure is not None:
            self.error = failure
            raise failure
        if int(flag.item()):
            self.error = ReplicaError(f"{int(flag.item())} other rank(s) of the replica failed in this step")
            raise self.error
        return worked

    def step(self) -> bool:
        self._leader_only()
        with self._lock:
            idle = not (self._pending or self.waiting or self.running or self.score_queue)
        if idle and time.monotonic() - self._last_tick < self.keepalive_s:
            return False
        return self._tick(step=True)

    def follow(self) -> None:
        """Follower ranks: mirror the leader until it shuts down."""
        if self.is_leader:
            raise RuntimeError("the leader drives the replica; only the other ranks follow")
        while not self._stop:
            self._tick(step=True)

    def shutdown(self) -> None:
        if self.is_leader:
            super().shutdown()                   # parks and joins the stepping thread, if any
            if self.error is None:               # after a failure the followers have already left follow()
                with self._step_lock:
                    self._tick(step=False, stop=True)
        else:
            self._stop = True
