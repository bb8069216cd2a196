"""Rollout engine on CPU: block manager, scheduler, prefix cache, adapters, pause/resume (reference runner)."""
import asyncio

import pytest
import torch

from art_b200.engine.engine import Engine, SamplingParams
from art_b200.engine.kv_cache import BlockManager
from art_b200.engine.runner import ReferenceRunner
from art_b200.models.config import PRESETS
from art_b200.models.weights import LoraConfig, init_base_weights, init_lora


def test_block_manager_alloc_free_and_prefix_cache():
    bm = BlockManager(8, 4, True)
    a = bm.alloc(3)
    assert len(a) == 3 and bm.num_free == 5
    assert bm.alloc(6) is None and bm.num_free == 5
    toks = list(range(12))
    bm.commit(a, toks, salt=7)
    bm.free(a)
    assert bm.num_free == 8                      # cached blocks stay evictable
    hit = bm.match_prefix(toks + [99], salt=7)
    assert hit == a                              # whole-block prefix re-used, same ids
    assert bm.match_prefix(toks, salt=8) == []   # other adapter salt: no reuse
    assert bm.match_prefix([0, 1, 2, 3, 9, 9, 9, 9], salt=7) == a[:1]
    bm.free(hit)
    bm.free(a[:1])
    got = bm.alloc(8)                            # eviction reclaims cached blocks when needed
    assert got is not None and sorted(got) == list(range(8))
    bm.free(got)
    bm.reset_prefix_cache()
    assert bm.match_prefix(toks, salt=7) == []
    assert bm.stats()["prefix_hits"] == 2


@pytest.fixture(scope="module")
def tiny():
    cfg = PRESETS["tiny"]
    base = init_base_weights(cfg, seed=0)
    return cfg, base


def make_engine(cfg, base, **kw):
    runner = ReferenceRunner(cfg, base, LoraConfig(), max_loras=2)
    bm = BlockManager(kw.pop("blocks", 64), 4, True)
    return Engine(runner, bm, eos_token_id=None, max_loras=2, **kw)


def test_greedy_is_deterministic_and_batching_invariant(tiny):
    cfg, base = tiny
    eng = make_engine(cfg, base, num_scheduler_steps=4)
    p = SamplingParams(max_tokens=6, temperature=0.0)
    a = eng.generate_sync([1, 2, 3, 4, 5], p)
    # same prompt again while another request shares the batch
    s1 = eng.add_request([1, 2, 3, 4, 5], p)
    s2 = eng.add_request([9, 8, 7], SamplingParams(max_tokens=3, temperature=0.0))
    while not (s1.finished and s2.finished):
        eng.step()
    assert a.output_ids == s1.output_ids and len(a.output_ids) == 6 and a.finish_reason == "length"
    assert len(s2.output_ids) == 3
    assert all(lp <= 0 for lp in a.logprobs)
    assert eng.bm.stats()["prefix_hits"] >= 1     # second request re-used the first one's prompt block


def test_adapter_changes_output_and_base_stays(tiny):
    cfg, base = tiny
    eng = make_engine(cfg, base)
    lora = init_lora(cfg, LoraConfig())
    g = torch.Generator().manual_seed(3)
    for k in lora:
        if "lora_B" in k:
            lora[k] = torch.randn(lora[k].shape, generator=g) * 0.5
    eng.set_adapter("my-model", lora)
    p = SamplingParams(max_tokens=5, temperature=0.0)
    base_out = eng.generate_sync([5, 6, 7, 8], p).output_ids
    lora_out = eng.generate_sync([5, 6, 7, 8], p, "my-model").output_ids
    assert base_out != lora_out
    assert eng.generate_sync([5, 6, 7, 8], p).output_ids == base_out
    with pytest.raises(KeyError):
        eng.add_request([1], p, "nope")


def test_preemption_when_blocks_run_out(tiny):
    cfg, base = tiny
    eng = make_engine(cfg, base, blocks=6, num_scheduler_steps=2)
    p = SamplingParams(max_tokens=10, temperature=0.0)
    seqs = [eng.add_request([i + 1, i + 2, i + 3], p) for i in range(3)]
    for _ in range(200):
        if all(s.finished for s in seqs):
            break
        eng.step()
    assert all(len(s.output_ids) == 10 for s in seqs)
    assert eng.stats.preemptions >= 1
    ref = make_engine(cfg, base)
    assert ref.generate_sync([1, 2, 3], p).output_ids == seqs[0].output_ids   # recompute after preemption is exact


def test_async_stream_pause_resume_and_abort(tiny):
    cfg, base = tiny
    eng = make_engine(cfg, base, num_scheduler_steps=1)
    eng.start()

    async def main():
        got = []
        async for ev in eng.generate([1, 2, 3], SamplingParams(max_tokens=4, temperature=1.0, seed=5)):
            got.append(ev.token_id)
            if len(got) == 2:
                eng.pause()
                assert not eng._run_gate.is_set()
                eng.resume()
        assert len(got) == 4
        # abort by abandoning the stream
        agen = eng.generate([4, 5, 6], SamplingParams(max_tokens=1000, temperature=0.0))
        await agen.__anext__()
        await agen.aclose()
        await asyncio.sleep(0.2)
        return got

    try:
        asyncio.run(main())
        for _ in range(100):
            if not eng.has_unfinished:
                break
            import time
            time.sleep(0.05)
        assert not eng.has_unfinished
    finally:
        eng.shutdown()


def test_complete_matches_the_token_stream_and_batches_events(tiny):
    """``Engine.complete`` returns the same tokens as the event stream; a multi-step decode hands a sequence its events
    of one scheduler step as one queue item."""
    cfg, base = tiny
    eng = make_engine(cfg, base, num_scheduler_steps=4)
    eng.start()
    p = SamplingParams(max_tokens=9, temperature=1.0, seed=11)

    async def main():
        streamed = [ev.token_id async for ev in eng.generate([1, 2, 3], p)]
        seq = await eng.complete([1, 2, 3], p)
        assert seq.output_ids == streamed and seq.finish_reason == "length" and len(seq.logprobs) == 9
        # per step, not per token: the first item is the prefill's token, later items hold up to four events
        s2 = eng.add_request([1, 2, 3], p, None, asyncio.get_running_loop())
        sizes = []
        while not (sizes and s2.finished and s2.queue.empty()):
            item = await s2.queue.get()
            sizes.append(len(item))
        assert sum(sizes) == 9 and max(sizes) > 1 and len(sizes) < 9
        # a cancelled caller aborts its request
        t = asyncio.ensure_future(eng.complete([7, 8, 9], SamplingParams(max_tokens=100000, temperature=0.0)))
        await asyncio.sleep(0.3)
        t.cancel()
        await asyncio.sleep(0.3)

    try:
        asyncio.run(main())
        import time
        for _ in range(100):
            if not eng.has_unfinished:
                break
            time.sleep(0.05)
        assert not eng.has_unfinished
    finally:
        eng.shutdown()


def test_top_k_top_p_restrict_the_support(tiny):
    from art_b200.ops.paged import reference_restrict

    x = torch.log(torch.tensor([0.4, 0.3, 0.15, 0.1, 0.05]))
    assert reference_restrict(x, 2, 1.0).tolist() == [True, True, False, False, False]
    assert reference_restrict(x, -1, 0.6).tolist() == [True, True, False, False, False]      # 0.4 + 0.3 reaches 0.6
    assert reference_restrict(x, -1, 0.75).tolist() == [True, True, True, False, False]
    assert reference_restrict(x, 3, 0.5).tolist() == [True, True, False, False, False]       # 0.5 of the top-3 mass 0.85
    assert reference_restrict(x, -1, 1.0).all()
    assert reference_restrict(x, -1, 1.0, 0.3).tolist() == [True, True, True, False, False]     # >= 0.3 * 0.4
    cfg, base = tiny
    eng = make_engine(cfg, base)
    greedy = eng.generate_sync([1, 2, 3, 4], SamplingParams(max_tokens=5, temperature=0.0))
    top1 = eng.generate_sync([1, 2, 3, 4], SamplingParams(max_tokens=5, temperature=1.3, top_k=1, seed=11))
    tiny_p = eng.generate_sync([1, 2, 3, 4], SamplingParams(max_tokens=5, temperature=1.3, top_p=1e-6, seed=12))
    assert top1.output_ids == greedy.output_ids and tiny_p.output_ids == greedy.output_ids
    free = eng.generate_sync([1, 2, 3, 4], SamplingParams(max_tokens=5, temperature=1.3, seed=11))
    assert all(lp <= 0 for lp in top1.logprobs + free.logprobs)


def test_kv_computed_under_replaced_adapter_is_not_reused(tiny):
    """A request in flight across pause -> set_adapter -> resume holds KV of the OLD weights; when it finishes its
    blocks must not enter the prefix cache under the new adapter version."""
    cfg, base = tiny
    eng = make_engine(cfg, base, num_scheduler_steps=1)
    g = torch.Generator().manual_seed(4)

    def rand_lora(scale):
        lora = init_lora(cfg, LoraConfig())
        for k in lora:
            if "lora_B" in k:
                lora[k] = torch.randn(lora[k].shape, generator=g) * scale
        return lora

    eng.set_adapter("m", rand_lora(0.5))
    prompt = list(range(1, 13))                      # three whole blocks of 4
    seq = eng.add_request(prompt, SamplingParams(max_tokens=6, temperature=0.0), "m")
    eng.step()                                       # prefill under version 1
    eng.step()
    assert not seq.finished
    eng.pause()
    eng.set_adapter("m", rand_lora(0.7))             # what ModelService.train does after a step
    eng.resume()
    while not seq.finished:
        eng.step()
    eng.step()                                       # releases the finished sequence
    slot = eng.adapters["m"]
    assert eng.bm.match_prefix(prompt, eng._salt(slot)) == []
    # a request that ran wholly under the new version is cached as before
    again = eng.generate_sync(prompt, SamplingParams(max_tokens=2, temperature=0.0), "m")
    eng.step()
    hit = eng.bm.match_prefix(prompt, eng._salt(slot))
    assert len(hit) == 3 and again.finished
    eng.bm.free(hit)


def test_chunked_prefill_splits_long_prompts_and_matches_unchunked(tiny):
    cfg, base = tiny
    p = SamplingParams(max_tokens=4, temperature=0.0)
    long_prompt = [(7 * i) % 900 + 1 for i in range(50)]
    short = [3, 4, 5]
    whole = make_engine(cfg, base, max_num_batched_tokens=4096).generate_sync(long_prompt, p).output_ids
    eng = make_engine(cfg, base, max_num_batched_tokens=16, num_scheduler_steps=1)      # 4-token blocks
    a = eng.add_request(long_prompt, p)
    b = eng.add_request(short, p)
    eng.step()
    # first step: a 16-token chunk of the long prompt; the short request waits for budget (FCFS)
    assert a in eng.prefilling and a.num_cached == 16 and not a.output_ids and eng.has_unfinished
    steps = 1
    while not (a.finished and b.finished):
        eng.step()
        steps += 1
        assert steps < 100
    assert a.output_ids == whole and len(b.output_ids) == 4
    assert eng.stats.prefill_steps >= 4 and not eng.prefilling        # 50 tokens at <= 16 per step
    assert eng.stats.prompt_tokens == 50 + 3
    # the last chunk shares its step with the short prompt when both fit the budget
    eng2 = make_engine(cfg, base, max_num_batched_tokens=16, num_scheduler_steps=1)
    a2 = eng2.add_request(long_prompt[:18], p)
    b2 = eng2.add_request(short, p)
    eng2.step()
    eng2.step()
    assert len(a2.output_ids) == 1 and len(b2.output_ids) == 1
    # an aborted request gives its blocks back half-way through its prompt
    eng3 = make_engine(cfg, base, max_num_batched_tokens=16, blocks=32)
    c = eng3.add_request(long_prompt, p)
    eng3.step()
    free_mid = eng3.bm.num_free
    eng3.abort(c)
    eng3.step()
    assert c.finished and c.finish_reason == "abort" and eng3.bm.num_free > free_mid and not eng3.has_unfinished
    # without chunking an oversized prompt runs whole, alone
    eng4 = make_engine(cfg, base, max_num_batched_tokens=16, enable_chunked_prefill=False)
    d = eng4.add_request(long_prompt, p)
    eng4.step()
    assert len(d.output_ids) == 1 and not eng4.prefilling


def test_prefix_cache_hits_are_budgeted_by_attended_tokens(tiny):
    """Sequences whose prompts hit the prefix cache bring few NEW tokens but many attended ones; one prefill step takes
    only as many of them as its attended-token budget (twice the batched-token budget) allows."""
    cfg, base = tiny
    eng = make_engine(cfg, base, max_num_batched_tokens=32, num_scheduler_steps=1, blocks=256)
    p = SamplingParams(max_tokens=2, temperature=0.0)
    prompt = [(3 * i) % 500 + 1 for i in range(41)]           # ten whole blocks of 4 + one token
    first = eng.generate_sync(prompt, p)
    eng.step()                                                # release -> the prompt's blocks enter the cache
    seqs = [eng.add_request(prompt, p) for _ in range(6)]     # each: 40 cached tokens, 1 new
    eng.step()
    started = [s for s in seqs if s.output_ids]
    assert 1 <= len(started) <= 2                             # 2 x 41 attended tokens > 64 stops the third
    while not all(s.finished for s in seqs):
        eng.step()
    assert all(s.output_ids == first.output_ids for s in seqs)


def test_a_closed_client_event_loop_does_not_stop_the_engine(tiny):
    """A request whose event loop went away (its process-level caller returned) only loses its own events: the
    stepping thread keeps serving the others."""
    cfg, base = tiny
    eng = make_engine(cfg, base, num_scheduler_steps=1)
    loop = asyncio.new_event_loop()
    orphan = eng.add_request([1, 2, 3], SamplingParams(max_tokens=3, temperature=0.0), None, loop)
    loop.close()
    eng.start()
    try:
        other = eng.generate_sync([4, 5, 6], SamplingParams(max_tokens=3, temperature=0.0))
        assert len(other.output_ids) == 3 and eng.error is None
        import time
        for _ in range(100):
            if orphan.finished:
                break
            time.sleep(0.05)
        assert orphan.finished and len(orphan.output_ids) == 3
    finally:
        eng.shutdown()


def test_engine_recovers_after_its_stepping_thread_failed(tiny):
    """A step that raises fails the requests in flight and stops the thread; the next request restarts the engine
    (blocks returned, prefix cache dropped) a bounded number of times."""
    cfg, base = tiny
    eng = make_engine(cfg, base, num_scheduler_steps=1)
    eng.start()
    real = eng.runner.decode
    state = {"fail": 1}

    def flaky(views, steps):
        if state["fail"] > 0:
            state["fail"] -= 1
            raise RuntimeError("injected step failure")
        return real(views, steps)

    eng.runner.decode = flaky
    try:
        async def first():
            with pytest.raises(RuntimeError, match="injected"):
                async for _ in eng.generate([1, 2, 3], SamplingParams(max_tokens=4, temperature=0.0)):
                    pass
        asyncio.run(first())
        for _ in range(100):
            if eng.error is not None:
                break
            time.sleep(0.02)
        assert eng.error is not None
        free_before = eng.bm.num_free
        seq = eng.generate_sync([1, 2, 3], SamplingParams(max_tokens=4, temperature=0.0))      # restarts the engine
        assert len(seq.output_ids) == 4 and eng.error is None and eng.recoveries == 1
        assert eng.bm.num_free >= free_before
        # the budget is finite
        eng.max_recoveries = 1
        state["fail"] = 1
        with pytest.raises(RuntimeError):
            eng.generate_sync([4, 5, 6], SamplingParams(max_tokens=4, temperature=0.0))
            eng.generate_sync([4, 5, 6], SamplingParams(max_tokens=4, temperature=0.0))
    finally:
        eng.shutdown()


def test_engine_logs_throughput_lines_unless_switched_off(tiny, caplog):
    import logging

    cfg, base = tiny
    eng = make_engine(cfg, base, num_scheduler_steps=1)
    eng.log_stats_interval = 0.0
    eng.start()
    try:
        with caplog.at_level(logging.INFO, logger="art_b200.engine.engine"):
            eng.generate_sync([1, 2, 3], SamplingParams(max_tokens=6, temperature=0.0))
        lines = [r.getMessage() for r in caplog.records if "generation throughput" in r.getMessage()]
        assert lines and "KV cache usage" in lines[0] and "prefix cache hit rate" in lines[0]
    finally:
        eng.shutdown()


def test_a_failing_prefill_reaches_the_request_that_was_being_prefilled(tiny):
    """A sequence is in no queue while the runner prefills it; if the runner raises there, the request must still be
    told (it used to wait for ever)."""
    cfg, base = tiny
    eng = make_engine(cfg, base, num_scheduler_steps=1)
    eng.start()

    def broken(views):
        raise RuntimeError("injected prefill failure")

    real = eng.runner.prefill
    eng.runner.prefill = broken
    try:
        async def main():
            with pytest.raises(RuntimeError, match="injected prefill"):
                await asyncio.wait_for(eng.complete([1, 2, 3], SamplingParams(max_tokens=4)), timeout=20)
        asyncio.run(main())
        with pytest.raises(ValueError, match="token ids"):
            eng.add_request(["input_ids", "attention_mask"], SamplingParams())
        eng.runner.prefill = real
        seq = eng.generate_sync([1, 2, 3], SamplingParams(max_tokens=4, temperature=0.0))       # recovers
        assert len(seq.output_ids) == 4
    finally:
        eng.shutdown()


def test_latency_statistics_in_the_metrics(tiny):
    cfg, base = tiny
    eng = make_engine(cfg, base, num_scheduler_steps=2)
    seqs = [eng.add_request([1, 2, 3 + i], SamplingParams(max_tokens=5, temperature=0.0)) for i in range(3)]
    while not all(s.finished for s in seqs):
        eng.step()
    m = eng.metrics()
    assert m["finished_requests"] == 3 and 0 < m["mean_time_to_first_token_s"] <= m["mean_request_s"]
