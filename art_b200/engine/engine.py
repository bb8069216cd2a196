"""Continuous-batching rollout engine.

A background thread owns the model runner and loops: admit waiting requests (prefill, with
prefix-cache reuse), otherwise advance every running sequence by up to ``num_scheduler_steps``
tokens in one device-side multi-step decode, then publish tokens to the per-request asyncio
queues.  ``pause()`` / ``resume()`` bracket a training phase: the loop stops at a step
boundary, in-flight requests keep their KV (or have it offloaded / discarded according to the
sleep level) and continue afterwards under whatever adapter weights are then loaded, which is
the observable behaviour of the reference's train/infer time-sharing
(``src/art/local/state.py:146-171``, ``src/art/local/vllm.py:115-145``) without its event-racing
gate.  Adapters are addressed by name (LoRA-by-name routing, ``src/art/dev/openai_server.py:17-23``);
loading one is a device-to-device copy into a slot (``service.py:164-174`` goes through disk).
"""
from __future__ import annotations

import asyncio
import itertools
import logging
import numbers
import threading
import os
import time
from collections import deque
from dataclasses import dataclass, field
from typing import AsyncIterator

from .kv_cache import BlockManager
from .runner import LogitProc, SeqView

log = logging.getLogger(__name__)


@dataclass
class SamplingParams:
    max_tokens: int = 16
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    min_p: float = 0.0
    n: int = 1
    stop: list[str] | None = None
    stop_token_ids: list[int] | None = None
    seed: int | None = None
    ignore_eos: bool = False
    guided_choice: list[str] | None = None
    top_logprobs: int = 0                  # alternatives reported per sampled token
    repetition_penalty: float = 1.0        # > 1 discourages tokens of prompt + output
    presence_penalty: float = 0.0          # subtracted once for every token already generated
    frequency_penalty: float = 0.0         # subtracted per occurrence in the output
    logit_bias: dict[int, float] | None = None
    stream_events: bool = True             # False: only the final event is delivered (see Engine.complete)
    include_stop_str_in_output: bool = False   # keep the matched stop string at the end of the returned text
    skip_special_tokens: bool = True       # the returned text leaves special tokens out (a matter of the server's decoding)
    min_tokens: int = 0                    # no end-of-sequence / stop token before this many tokens
    allowed_token_ids: list[int] | None = None   # only these ids may be drawn
    bad_words_ids: list[list[int]] | None = None  # token sequences that must not appear in the output
    guided_regex: str | None = None        # the completion's text has to match this expression (engine/grammar.py);
                                           # needs Engine.token_masker (the server sets it from its tokenizer)

    @property
    def needs_logits(self) -> bool:
        return (self.top_logprobs > 0 or self.repetition_penalty != 1.0 or self.presence_penalty != 0.0
                or self.frequency_penalty != 0.0 or bool(self.logit_bias) or self.guided_regex is not None
                or self.min_tokens > 0 or bool(self.allowed_token_ids) or bool(self.bad_words_ids))


@dataclass(slots=True)
class TokenEvent:
    token_id: int
    logprob: float
    finished: bool = False
    finish_reason: str | None = None
    top_logprobs: list[tuple[int, float]] | None = None
    cached_tokens: int | None = None      # on the last event: prompt tokens whose KV came from the prefix cache


class Sequence:
    _ids = itertools.count(1)

    def __init__(self, prompt_ids: list[int], params: SamplingParams, adapter: int, loop: asyncio.AbstractEventLoop | None):
        self.id = next(Sequence._ids)
        self.prompt_ids = list(prompt_ids)
        self.output_ids: list[int] = []
        self._tokens: list[int] = list(prompt_ids)     # prompt + output, grown in place (read-only for everyone else)
        self.logprobs: list[float] = []
        self.params = params
        self.adapter = adapter
        self.blocks: list[int] = []
        self.num_cached = 0
        self.prefix_hit_tokens = 0            # prompt tokens served from the prefix cache at (the last) admission
        self.salt: int | None = None          # prefix-cache salt (adapter slot + version) the KV was computed under
        self.finished = False
        self.finish_reason: str | None = None
        self.aborted = False
        self.loop = loop
        self.queue: asyncio.Queue | None = asyncio.Queue() if loop is not None else None
        self.seed = params.seed if params.seed is not None else (self.id * 2654435761) & 0x7FFFFFFF
        self.arrival = time.monotonic()
        self.forced: deque[int] = deque()     # guided decoding: tokens to emit verbatim
        self.top_logprobs: list = []          # per generated token: None or [(token, logprob)] (when requested)
        self.proc = (LogitProc(len(self.prompt_ids), params.repetition_penalty, params.presence_penalty,
                               params.frequency_penalty, params.logit_bias, params.top_logprobs,
                               min_tokens=params.min_tokens, bad_words_ids=params.bad_words_ids)
                     if params.needs_logits else None)
        self.done_event = threading.Event()

    @property
    def tokens(self) -> list[int]:
        """Prompt followed by the tokens generated so far: one list that grows in place (the scheduler asks for it
        several times per sequence and step; callers must not modify it)."""
        return self._tokens

    def view(self) -> SeqView:
        return SeqView(self.tokens, self.num_cached, self.blocks, self.adapter, self.params.temperature, self.seed,
                       len(self.output_ids), self.params.top_p, self.params.top_k, self.params.min_p, self.proc)


def _deliver(per_queue: dict) -> None:
    """Runs on the event loop: hands every sequence the token events of one scheduler step."""
    for q, events in per_queue.items():
        q.put_nowait(events)


@dataclass
class EngineStats:
    prompt_tokens: int = 0
    generated_tokens: int = 0
    prefill_steps: int = 0
    decode_steps: int = 0
    preemptions: int = 0
    finished_requests: int = 0
    ttft_s: float = 0.0         # sum over requests: arrival -> first token
    request_s: float = 0.0      # sum over finished requests: arrival -> last token
    runner_s: float = 0.0       # wall time inside runner.prefill / runner.decode (device work + its host staging)
    step_s: float = 0.0         # wall time of scheduler steps that did work (runner time included)
    started: float = field(default_factory=time.monotonic)


class Engine:
    def __init__(self, runner, block_manager: BlockManager, *, eos_token_id: int | None, max_num_seqs: int = 256,
                 max_num_batched_tokens: int = 16384, num_scheduler_steps: int = 16, max_model_len: int = 32768,
                 max_loras: int = 4, kv_cache=None, enable_chunked_prefill: bool = True,
                 log_stats_interval: float | None = None):
        """``max_num_batched_tokens`` bounds the new tokens of one prefill step.  With ``enable_chunked_prefill`` a
        prompt longer than what is left of that budget is computed over several steps, a block-aligned chunk at a
        time (its KV accumulates in its blocks; the token is sampled after the last chunk), so a long prompt neither
        waits for an empty step nor builds one oversized forward pass; without it such a prompt runs alone, whole."""
        self.runner, self.bm, self.kv = runner, block_manager, kv_cache
        self.log_stats_interval = log_stats_interval     # seconds between throughput lines in the log; None: no lines
        self._stats_mark = (time.monotonic(), 0, 0, 0, 0)   # time, prompt tokens, generated tokens, cache queries, hits
        self.chunked = enable_chunked_prefill
        self.prefilling: list[Sequence] = []      # admitted, prompt KV partly computed
        self.eos = eos_token_id
        self.max_num_seqs, self.max_batched = max_num_seqs, max_num_batched_tokens
        self.n_steps, self.max_model_len = max(1, num_scheduler_steps), max_model_len
        self.waiting: deque[Sequence] = deque()
        self.running: list[Sequence] = []
        self._outbox: dict = {}     # event loop -> {queue: [TokenEvent, ...]} of the scheduler step in progress
        self._inflight: list = []   # sequences handed to the runner for prefill (in no queue meanwhile)
        self.token_masker = None    # grammar.TokenMasker of the serving tokenizer: enables SamplingParams.guided_regex
        self.max_recoveries = 3     # automatic restarts of the stepping thread after an error (see recover())
        self.recoveries = 0
        self.score_queue: deque = deque()
        self.adapters: dict[str, int] = {}
        self.adapter_version = [0] * max_loras
        self.max_loras = max_loras
        self.stats = EngineStats()
        self._trace, self._trace_steps = None, 0
        self._lock = threading.Lock()
        self._wake = threading.Event()
        self._run_gate = threading.Event()
        self._run_gate.set()
        self._step_lock = threading.Lock()
        self._stop = False
        self._thread: threading.Thread | None = None
        self.error: BaseException | None = None

    # -- adapters ---------------------------------------------------------------------------------
    def set_adapter(self, name: str, state: dict | None) -> int:
        """Load (or replace) the adapter served under ``name``; returns its slot.  Call while paused or idle."""
        if name in self.adapters:
            slot = self.adapters[name]
        else:
            used = set(self.adapters.values())
            free = [s for s in range(self.max_loras) if s not in used]
            if not free:
                raise RuntimeError(f"all {self.max_loras} adapter slots are in use")
            slot = free[0]
            self.adapters[name] = slot
        self.runner.set_adapter(slot, state)
        self.adapter_version[slot] += 1   # new salt: KV computed under the old weights is not reused
        return slot

    def remove_adapter(self, name: str) -> None:
        slot = self.adapters.pop(name, None)
        if slot is not None:
            self.runner.set_adapter(slot, None)
            self.adapter_version[slot] += 1

    def set_vocabulary(self, vocab: list[bytes], eos_token_id: int | None = None) -> None:
        """The byte string of every token id (``grammar.vocabulary_bytes``): builds the allowed-token index that
        ``SamplingParams.guided_regex`` needs."""
        from .grammar import TokenMasker

        self.token_masker = TokenMasker(vocab, self.eos if eos_token_id is None else eos_token_id)

    def _salt(self, adapter: int) -> int:
        return 0x51 if adapter < 0 else (adapter + 1) * 1_000_003 + self.adapter_version[adapter]

    # -- lifecycle --------------------------------------------------------------------------------
    def start(self) -> None:
        if self._thread is None:
            self._thread = threading.Thread(target=self._loop, name="art-b200-engine", daemon=True)
            self._thread.start()

    def shutdown(self) -> None:
        self._stop = True
        self._run_gate.set()
        self._wake.set()
        if self._thread is not None:
            self._thread.join(timeout=10)
            self._thread = None

    def pause(self, timeout: float = 600.0) -> None:
        """Stop stepping at the next step boundary and wait until the loop is parked."""
        self._run_gate.clear()
        self._wake.set()
        if not self._step_lock.acquire(timeout=timeout):   # waits for the step in progress, if any
            raise TimeoutError("engine did not reach a step boundary")
        self._step_lock.release()

    def resume(self) -> None:
        self._run_gate.set()
        self._wake.set()

    @property
    def has_unfinished(self) -> bool:
        with self._lock:
            return bool(self.waiting or self.running or self.prefilling)

    def sleep(self, level: int = 1) -> None:
        """Release KV memory while paused: level 1 keeps contents on the host when requests are in
        flight, level 2 discards (and forgets the prefix cache)."""
        if self.kv is None:
            return
        if getattr(self.kv, "arena", None) is None and hasattr(self.runner, "drop_graphs"):
            # without the address-stable arena the cache comes back at new addresses: captured decode graphs
            # would replay against freed memory
            self.runner.drop_graphs()
        if level == 1 and self.has_unfinished:
            self.kv.offload()
        else:
            self.reset_prefix_cache()
            self.kv.discard()
            with self._lock:   # KV of in-flight sequences is gone: recompute them from their tokens
                for s in self.running + self.prefilling:
                    self.bm.free(s.blocks)
                    s.blocks, s.num_cached = [], 0
                    self.waiting.appendleft(s)
                self.running, self.prefilling = [], []

    def wake_up(self) -> None:
        if self.kv is not None:
            self.kv.restore()

    def reset_prefix_cache(self) -> None:
        self.bm.reset_prefix_cache()

    # -- requests ---------------------------------------------------------------------------------
    def add_request(self, prompt_ids: list[int], params: SamplingParams, adapter_name: str | None = None,
                    loop: asyncio.AbstractEventLoop | None = None) -> Sequence:
        seq = self._new_sequence(prompt_ids, params, adapter_name, loop)
        with self._lock:
            self.waiting.append(seq)
        self._wake.set()
        return seq

    def _new_sequence(self, prompt_ids: list[int], params: SamplingParams, adapter_name: str | None,
                      loop: asyncio.AbstractEventLoop | None) -> Sequence:
        """Validate a request and build its sequence (not yet queued)."""
        if self.error is not None:
            # a request arriving after a failure restarts the engine, a bounded number of times (a failure that comes
            # back every time is a bug to look at, not something to loop on)
            if self.recoveries < self.max_recoveries and self._thread is not None:
                self.recover()
            else:
                raise RuntimeError("engine stopped after an error") from self.error
        if len(prompt_ids) == 0 or not all(isinstance(t, numbers.Integral) for t in prompt_ids):
            raise ValueError("a prompt is a non-empty list of token ids")
        if len(prompt_ids) + 1 > self.max_model_len:
            raise ValueError(f"prompt of {len(prompt_ids)} tokens exceeds max_model_len={self.max_model_len}")
        adapter = -1
        if adapter_name is not None:
            if adapter_name not in self.adapters:
                raise KeyError(f"unknown adapter {adapter_name!r}")
            adapter = self.adapters[adapter_name]
        seq = Sequence(prompt_ids, params, adapter, loop)
        if seq.proc is not None and params.min_tokens > 0:
            seq.proc.end_ids = tuple(([self.eos] if self.eos is not None and not params.ignore_eos else [])
                                     + list(params.stop_token_ids or []))
        if params.allowed_token_ids:
            if params.guided_regex is not None:
                raise ValueError("allowed_token_ids and guided_regex exclude each other")
            from .grammar import AllowedSet

            seq.proc.grammar = AllowedSet(params.allowed_token_ids)
        if params.guided_regex is not None:
            if self.token_masker is None:
                raise ValueError("guided_regex needs Engine.token_masker (a grammar.TokenMasker over the tokenizer's vocabulary)")
            from .grammar import GrammarState, compile_cached

            seq.proc.grammar = GrammarState(compile_cached(params.guided_regex), self.token_masker)
        return seq

    def abort(self, seq: Sequence) -> None:
        seq.aborted = True
        self._wake.set()

    async def generate_steps(self, prompt_ids: list[int], params: SamplingParams, adapter_name: str | None = None
                             ) -> AsyncIterator[list[TokenEvent]]:
        """Async stream of one request's sampled tokens, grouped as the scheduler produced them: one list per scheduler
        step (up to ``num_scheduler_steps`` tokens).  Cancelling the consumer aborts the request."""
        seq = self.add_request(prompt_ids, params, adapter_name, asyncio.get_running_loop())
        try:
            while True:
                item = await seq.queue.get()
                if isinstance(item, BaseException):
                    raise item
                events = item if isinstance(item, list) else [item]
                for k, ev in enumerate(events):
                    if ev.finished:
                        events = events[:k + 1]
                        break
                yield events
                if events and events[-1].finished:
                    return
        finally:
            if not seq.finished:
                self.abort(seq)

    async def generate(self, prompt_ids: list[int], params: SamplingParams, adapter_name: str | None = None
                       ) -> AsyncIterator[TokenEvent]:
        """Async stream of sampled tokens for one request; cancelling the consumer aborts the request."""
        agen = self.generate_steps(prompt_ids, params, adapter_name)
        try:
            async for events in agen:
                for ev in events:
                    yield ev
        finally:
            await agen.aclose()

    async def complete(self, prompt_ids: list[int], params: SamplingParams, adapter_name: str | None = None) -> Sequence:
        """Runs one request to its end and returns its sequence (``output_ids``, ``logprobs``, ``top_logprobs``,
        ``finish_reason``).  No per-token events cross threads: a non-streaming HTTP request costs the event loop one
        wake-up instead of one per token.  Cancelling the caller aborts the request."""
        import dataclasses

        seq = self.add_request(prompt_ids, dataclasses.replace(params, stream_events=False), adapter_name,
                               asyncio.get_running_loop())
        try:
            while True:
                item = await seq.queue.get()
                if isinstance(item, BaseException):
                    raise item
                if seq.finished:
                    return seq
        finally:
            if not seq.finished:
                self.abort(seq)

    async def score(self, prompt_ids: list[int], completion_ids: list[int], adapter_name: str | None = None) -> list[float]:
        """Per-token log-probabilities of ``completion_ids`` after ``prompt_ids`` (teacher forcing)."""
        adapter = -1 if adapter_name is None else self.adapters[adapter_name]
        loop = asyncio.get_running_loop()
        fut = loop.create_future()
        with self._lock:
            self.score_queue.append((list(prompt_ids) + list(completion_ids), len(prompt_ids), adapter, loop, fut))
        self._wake.set()
        if self._thread is None:
            self.step()
        return await fut

    def generate_sync(self, prompt_ids: list[int], params: SamplingParams, adapter_name: str | None = None) -> Sequence:
        """Blocking helper (tests, benchmarks): drives the loop inline if no thread is running."""
        seq = self.add_request(prompt_ids, params, adapter_name, None)
        if self._thread is None:
            while not seq.finished:
                self.step()
        else:
            seq.done_event.wait()
        return seq

    # -- scheduling -------------------------------------------------------------------------------
    def _emit(self, seq: Sequence, tok: int, lp: float, top=None) -> None:
        seq.output_ids.append(tok)
        seq._tokens.append(tok)
        seq.logprobs.append(lp)
        seq.top_logprobs.append(top)
        self.stats.generated_tokens += 1
        p = seq.params
        reason = None
        grammar = seq.proc.grammar if seq.proc is not None else None
        if grammar is not None:
            grammar.advance(tok)
        if grammar is not None and (grammar.exhausted or (self.eos is not None and tok == self.eos)):
            reason = "stop"         # nothing can follow (or the automaton accepted and the model ended the text)
        elif not p.ignore_eos and self.eos is not None and tok == self.eos:
            reason = "stop"
        elif p.stop_token_ids and tok in p.stop_token_ids:
            reason = "stop"
        elif len(seq.output_ids) >= p.max_tokens or len(seq.prompt_ids) + len(seq.output_ids) >= self.max_model_len:
            reason = "length"
        if len(seq.output_ids) == 1:
            self.stats.ttft_s += time.monotonic() - seq.arrival
        if reason:
            seq.finished, seq.finish_reason = True, reason
            self.stats.finished_requests += 1
            self.stats.request_s += time.monotonic() - seq.arrival
        if seq.loop is not None and (p.stream_events or seq.finished):
            # delivered by _flush_events at the end of the scheduler step: one wake-up of the event loop per step and
            # one queue item per sequence, however many sequences and decode steps the step covered
            self._outbox.setdefault(seq.loop, {}).setdefault(seq.queue, []).append(
                TokenEvent(tok, lp, seq.finished, reason, top, seq.prefix_hit_tokens if seq.finished else None))

    def _flush_events(self) -> None:
        if not self._outbox:
            return
        outbox, self._outbox = self._outbox, {}
        for loop, per_queue in outbox.items():
            try:
                loop.call_soon_threadsafe(_deliver, per_queue)
            except RuntimeError:
                pass        # that client's event loop is closed: nobody is left to read its events; the others go on

    def _release(self, seq: Sequence) -> None:
        if seq.blocks:
            toks = seq.tokens
            # KV computed (even partly) under weights that were replaced since admission must not become reusable
            if seq.salt is not None and seq.salt == self._salt(seq.adapter):
                self.bm.commit(seq.blocks, toks[: len(toks) - 1], seq.salt)
            self.bm.free(seq.blocks)
            seq.blocks = []
        seq.done_event.set()

    def _blocks_needed(self, n_tokens: int) -> int:
        bs = self.bm.block_size
        return (n_tokens + bs - 1) // bs

    def _admit(self) -> list[tuple[Sequence, int]]:
        """Work of one prefill step: ``(sequence, upto)`` pairs, ``upto`` = prompt tokens computed after the step.
        Partly prefilled sequences go first, then waiting ones FCFS; bounded by the token budget, the sequence limit
        and free blocks."""
        picked: list[tuple[Sequence, int]] = []
        budget = self.max_batched
        # tokens attended in the step (cached prefix + new): the prefill gathers the cached K/V of every picked sequence
        # into one dense buffer, so many prefix-cache hits with long prefixes must not all land in the same step
        att_budget = 2 * self.max_batched
        bs = self.bm.block_size

        def chunk(n_new: int) -> int:
            """How many of ``n_new`` missing tokens fit this step (0: none)."""
            if n_new <= budget:
                return n_new
            if self.chunked:
                return budget // bs * bs
            return n_new if not picked else 0          # unchunked: an oversized prompt runs alone

        for seq in self.prefilling:
            take = chunk(len(seq.tokens) - seq.num_cached)
            if take <= 0 or (picked and seq.num_cached + take > att_budget):
                break
            picked.append((seq, seq.num_cached + take))
            budget -= take
            att_budget -= seq.num_cached + take
        with self._lock:
            while self.waiting and budget > 0 and len(self.running) + len(self.prefilling) + \
                    sum(1 for s, _ in picked if s not in self.prefilling) < self.max_num_seqs:
                seq = self.waiting[0]
                if seq.aborted:
                    self.waiting.popleft()
                    seq.finished, seq.finish_reason = True, "abort"
                    seq.done_event.set()
                    continue
                toks = seq.tokens
                salt = self._salt(seq.adapter)
                cached = self.bm.match_prefix(toks[:-1], salt)   # always recompute the last token
                n_new = len(toks) - len(cached) * bs
                take = chunk(n_new)
                if take <= 0 or (picked and len(cached) * bs + take > att_budget):
                    self.bm.free(cached)
                    break
                need = self._blocks_needed(len(toks) + 1) - len(cached)
                fresh = self.bm.alloc(need)
                if fresh is None:
                    self.bm.free(cached)
                    break
                self.waiting.popleft()
                seq.blocks = cached + fresh
                seq.num_cached = len(cached) * bs
                seq.prefix_hit_tokens = min(seq.num_cached, len(seq.prompt_ids))
                seq.salt = salt
                picked.append((seq, seq.num_cached + take))
                budget -= take
                att_budget -= seq.num_cached + take
        return picked

    def _ensure_decode_blocks(self, steps: int) -> int:
        """Give every running sequence room for ``steps`` more tokens; preempt the newest if needed."""
        while True:
            steps = max(1, steps)
            short = []
            for s in self.running:
                need = self._blocks_needed(len(s.tokens) + steps) - len(s.blocks)
                if need > 0:
                    short.append((s, need))
            total = sum(n for _, n in short)
            if total <= self.bm.num_free:
                for s, n in short:
                    s.blocks += self.bm.alloc(n)
                return steps
            if steps > 1:
                steps = 1
                continue
            victim = self.running.pop()   # newest: recompute later
            self.bm.free(victim.blocks)
            victim.blocks, victim.num_cached = [], 0
            with self._lock:
                self.waiting.appendleft(victim)
            self.stats.preemptions += 1
            if not self.running:
                return 0

    def step(self) -> bool:
        """One scheduler iteration.  Returns False when there was nothing to do."""
        t0 = time.monotonic()
        worked = False
        try:
            worked = self._step()
            return worked
        finally:
            self._flush_events()
            if worked:
                self.stats.step_s += time.monotonic() - t0

    def _step(self) -> bool:
        while self.score_queue:
            with self._lock:
                toks, n_prompt, adapter, loop, fut = self.score_queue.popleft()
            try:
                res = self.runner.score(toks, n_prompt, adapter)
                reply = lambda f=fut, r=res: f.done() or f.set_result(r)      # noqa: E731
            except BaseException as e:  # noqa: BLE001
                reply = lambda f=fut, e=e: f.done() or f.set_exception(e)     # noqa: E731
            try:
                loop.call_soon_threadsafe(reply)
            except RuntimeError:
                pass        # the caller's event loop is closed
        for s in [s for s in self.running + self.prefilling if s.aborted and not s.finished]:
            s.finished, s.finish_reason = True, "abort"
        for s in [s for s in self.prefilling if s.finished]:    # aborted half-way through its prompt
            self.prefilling.remove(s)
            self.bm.free(s.blocks)
            s.blocks = []
            s.done_event.set()
        done = [s for s in self.running if s.finished]
        if done:
            self.running = [s for s in self.running if not s.finished]
            for s in done:
                self._release(s)
        work = self._admit()
        if work:
            self.stats.prefill_steps += 1
            self.stats.prompt_tokens += sum(upto - s.num_cached for s, upto in work)
            views = []
            for s, upto in work:
                v = s.view()
                v.upto = upto
                views.append(v)
            t0 = time.monotonic()
            self._inflight = [s for s, _ in work]       # out of the queues while the runner works: told if it fails
            toks, lps = self.runner.prefill(views)
            self._inflight = []
            self.stats.runner_s += time.monotonic() - t0
            tops = getattr(self.runner, "last_top_logprobs", None)
            for i, (s, upto) in enumerate(work):
                if upto < len(s.tokens):                # more chunks to come: the KV so far stays in its blocks
                    s.num_cached = upto
                    if s not in self.prefilling:
                        self.prefilling.append(s)
                    continue
                if s in self.prefilling:
                    self.prefilling.remove(s)
                t = toks[i]
                if s.forced:
                    t = s.forced.popleft()
                s.num_cached = 0
                self._emit(s, t, lps[i], tops[0][i] if tops else None)
                self.running.append(s)
            return True
        if not self.running:
            return False
        remaining = min(s.params.max_tokens - len(s.output_ids) for s in self.running)
        steps = self._ensure_decode_blocks(min(self.n_steps, max(1, remaining)))
        if steps == 0 or not self.running:
            return True
        if any(s.forced or s.proc is not None for s in self.running):
            steps = 1      # the next step's input (forced token, penalties) depends on the host
        self.stats.decode_steps += steps
        t0 = time.monotonic()
        toks, lps = self.runner.decode([s.view() for s in self.running], steps)
        self.stats.runner_s += time.monotonic() - t0
        tops = getattr(self.runner, "last_top_logprobs", None)
        for k in range(steps):
            for i, s in enumerate(self.running):
                if s.finished:
                    continue
                t = toks[k][i]
                if s.forced:
                    t = s.forced.popleft()
                self._emit(s, t, lps[k][i], tops[k][i] if tops else None)
        return True

    def _traced_step(self) -> bool:
        """``step()``; with ``ARTB_TRACE_FILE`` set every iteration becomes a span of a Chrome trace plus counters
        (running / waiting sequences, free KV blocks), saved every 200 steps and on shutdown."""
        path = os.environ.get("ARTB_TRACE_FILE")
        if not path:
            return self.step()
        if self._trace is None:
            from ..utils.profiling import ChromeTrace

            self._trace = ChromeTrace("art_b200.engine")
        n_run, n_wait = len(self.running), len(self.waiting)
        with self._trace.span("engine.step", cat="scheduler", running=n_run, waiting=n_wait):
            worked = self.step()
        if worked:
            self._trace.counter("sequences", running=len(self.running), waiting=len(self.waiting))
            self._trace.counter("kv_blocks", free=self.bm.num_free)
            self._trace_steps += 1
            if self._trace_steps % 200 == 0:
                self._trace.save(path)
        return worked

    def _loop(self) -> None:
        try:
            dev = getattr(self.runner, "device", None)
            if dev is not None and getattr(dev, "type", "cpu") == "cuda":
                import torch

                torch.cuda.set_device(dev)      # the current device is per thread and starts at 0
            while not self._stop:
                self._run_gate.wait()
                with self._step_lock:
                    if self._stop or not self._run_gate.is_set():
                        continue
                    worked = self._traced_step()
                if self.log_stats_interval is not None:
                    self._log_stats()
                if not worked:
                    self._wake.wait(timeout=0.05)
                    self._wake.clear()
        except BaseException as e:  # noqa: BLE001 - report to every waiter, then stop
            self.error = e
            with self._lock:
                seqs = list(self.waiting) + self.running + self.prefilling
            seqs += [s for s in self._inflight if s not in seqs]
            self._inflight = []
            for s in seqs:
                if s.loop is not None:
                    try:
                        s.loop.call_soon_threadsafe(s.queue.put_nowait, e)
                    except RuntimeError:
                        pass            # closed event loop
                s.finished = True
                s.done_event.set()

    def _log_stats(self) -> None:
        """One throughput line per ``log_stats_interval`` seconds in which tokens were processed (what the reference's
        engine prints unless ``disable_log_stats`` is set)."""
        now = time.monotonic()
        t0, p0, g0, q0, h0 = self._stats_mark
        if now - t0 < self.log_stats_interval:
            return
        st = self.bm.stats()
        p, g = self.stats.prompt_tokens, self.stats.generated_tokens
        q, h = st.get("prefix_queries", 0), st.get("prefix_hits", 0)
        self._stats_mark = (now, p, g, q, h)
        if p == p0 and g == g0 and not self.running and not self.waiting:
            return
        dt = now - t0
        log.info("prompt throughput %.1f tokens/s, generation throughput %.1f tokens/s, running %d, waiting %d, "
                 "KV cache usage %.1f %%, prefix cache hit rate %.1f %%, preemptions %d",
                 (p - p0) / dt, (g - g0) / dt, len(self.running), len(self.waiting),
                 100.0 * (1.0 - self.bm.num_free / self.bm.num_blocks), 100.0 * (h - h0) / max(1, q - q0),
                 self.stats.preemptions)

    def recover(self) -> bool:
        """Bring the engine back after its stepping thread stopped on an error: every request that was in flight has
        already been failed; their blocks are returned, the prefix cache and the captured graphs are dropped (their
        contents may be half written), and a new stepping thread starts.  Returns False when there was nothing to
        recover from.  Adapters and weights stay as they are."""
        if self.error is None:
            return False
        t, self._thread = self._thread, None
        if t is not None:
            t.join(timeout=10)
        with self._lock:
            dead = list(self.waiting) + self.running + self.prefilling
            self.waiting.clear()
            self.running, self.prefilling = [], []
        for s in dead:
            if s.blocks:
                self.bm.free(s.blocks)
                s.blocks = []
        self.bm.reset_prefix_cache()
        self._outbox = {}
        drop = getattr(self.runner, "drop_graphs", None)
        if drop is not None:
            drop()
        self.recoveries = self.recoveries + 1
        self.error = None
        self._stop = False
        self._run_gate.set()
        self.start()
        return True

    def metrics(self) -> dict:
        st = self.bm.stats()
        dt = max(1e-9, time.monotonic() - self.stats.started)
        return {"running": len(self.running), "waiting": len(self.waiting), "prompt_tokens": self.stats.prompt_tokens,
                "generated_tokens": self.stats.generated_tokens, "preemptions": self.stats.preemptions,
                "recoveries": self.recoveries, "finished_requests": self.stats.finished_requests,
                "mean_time_to_first_token_s": self.stats.ttft_s / max(1, self.stats.finished_requests + len(self.running)),
                "mean_request_s": self.stats.request_s / max(1, self.stats.finished_requests),
                "kv_free_blocks": self.bm.num_free, "kv_total_blocks": self.bm.num_blocks,
                "kv_utilisation": 1.0 - self.bm.num_free / self.bm.num_blocks, "tokens_per_s": self.stats.generated_tokens / dt,
                "decode_steps": self.stats.decode_steps, "prefill_steps": self.stats.prefill_steps,
                "runner_seconds": round(self.stats.runner_s, 3), "step_seconds": round(self.stats.step_s, 3), **st}
