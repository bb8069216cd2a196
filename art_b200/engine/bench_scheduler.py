"""Host-side cost of the rollout engine's scheduler: ``python -m art_b200.engine.bench_scheduler``.

The engine runs with a runner that returns tokens at once, so what is measured is admission, block allocation,
per-token bookkeeping and event delivery alone (no GPU, no model).  Compare the tokens per second printed here with the
decode throughput of the device (``engine/bench_decode.py``): the ratio is the share of a decode step the scheduler
can cost at most when it is not overlapped with the device.  ``--http N`` puts the completion server in front and sends
N concurrent chat requests over the loopback interface (``--stream`` for event streams).
"""
from __future__ import annotations

import argparse
import json
import random
import time

from .engine import Engine, SamplingParams
from .kv_cache import BlockManager


class InstantRunner:
    """The runner interface with no work behind it."""

    last_top_logprobs = None

    def prefill(self, seqs):
        return [7] * len(seqs), [-1.0] * len(seqs)

    def decode(self, seqs, n_steps):
        n = len(seqs)
        return [[7] * n for _ in range(n_steps)], [[-1.0] * n for _ in range(n_steps)]

    def set_adapter(self, slot, state):
        pass


def run(seqs: int = 512, prompt_len: int = 1000, new_tokens: int = 1000, scheduler_steps: int = 16,
        prefix_caching: bool = False) -> dict:
    bs = 16
    eng = Engine(InstantRunner(), BlockManager(seqs * ((prompt_len + new_tokens) // bs + 2), bs, prefix_caching),
                 eos_token_id=None, max_num_seqs=seqs, max_num_batched_tokens=32768, num_scheduler_steps=scheduler_steps,
                 max_model_len=prompt_len + new_tokens + 16)
    rng = random.Random(0)
    reqs = [eng.add_request([rng.randrange(1000) for _ in range(prompt_len)],
                            SamplingParams(max_tokens=new_tokens, stream_events=False)) for _ in range(seqs)]
    t0 = time.perf_counter()
    iters = 0
    while not all(s.finished for s in reqs):
        eng.step()
        iters += 1
    dt = time.perf_counter() - t0
    return {"op": "scheduler_only", "seqs": seqs, "prompt_len": prompt_len, "new_tokens": new_tokens,
            "scheduler_steps": scheduler_steps, "prefix_caching": prefix_caching, "seconds": round(dt, 3),
            "iterations": iters, "ms_per_iteration": round(dt / iters * 1e3, 3),
            "us_per_decode_step": round(dt / (iters * scheduler_steps) * 1e6, 1),
            "tokens_per_s": round(seqs * new_tokens / dt)}


async def run_http(requests: int = 800, prompt_tokens: int = 1000, new_tokens: int = 1000, stream: bool = False,
                   scheduler_steps: int = 16, max_num_seqs: int = 512) -> dict:
    """The same instant runner behind the completion server, driven over HTTP on the loopback interface: what the
    server, the event delivery and the JSON encoding cost per request and per token when the model costs nothing."""
    import asyncio
    import socket

    import httpx

    from ..local.tokenizer import ByteChatTokenizer
    from .server import OpenAIServer, serve

    tok = ByteChatTokenizer(512)
    bs = 16
    eng = Engine(InstantRunner(), BlockManager(max_num_seqs * ((prompt_tokens + new_tokens) // bs + 8), bs, False),
                 eos_token_id=None, max_num_seqs=max_num_seqs, max_num_batched_tokens=32768,
                 num_scheduler_steps=scheduler_steps, max_model_len=prompt_tokens + new_tokens + 64)
    eng.start()
    srv = OpenAIServer(eng, tok, "instant", api_key=None)
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    ready = asyncio.Event()
    task = asyncio.create_task(serve(srv, "127.0.0.1", port, ready=ready))
    await ready.wait()
    prompt = "x" * max(1, prompt_tokens - 30)          # the chat template adds about 30 tokens
    body = {"model": "instant", "messages": [{"role": "user", "content": prompt}], "max_tokens": new_tokens, "stream": stream}
    try:
        limits = httpx.Limits(max_connections=requests, max_keepalive_connections=requests)
        async with httpx.AsyncClient(timeout=600, limits=limits) as c:
            async def one():
                if not stream:
                    r = await c.post(f"http://127.0.0.1:{port}/v1/chat/completions", json=body)
                    return r.json()["usage"]["completion_tokens"]
                n = 0
                async with c.stream("POST", f"http://127.0.0.1:{port}/v1/chat/completions", json=body) as r:
                    async for line in r.aiter_lines():
                        if line.startswith("data: {"):
                            n += line.count('"token":')          # a chunk carries the tokens of one scheduler step
                return n

            await asyncio.gather(*[one() for _ in range(min(8, requests))])      # warm-up: imports, connection pool
            t0 = time.perf_counter()
            done = await asyncio.gather(*[one() for _ in range(requests)])
            dt = time.perf_counter() - t0
    finally:
        task.cancel()
        try:
            await task
        except BaseException:  # noqa: BLE001
            pass
        eng.shutdown()
    return {"op": "http_instant_runner", "requests": requests, "prompt_tokens": prompt_tokens, "new_tokens": new_tokens,
            "stream": stream, "seconds": round(dt, 2), "requests_per_s": round(requests / dt, 1),
            "completion_tokens_per_s": round(sum(done) / dt), "completion_tokens": sum(done)}


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--seqs", type=int, default=512)
    ap.add_argument("--prompt-len", type=int, default=1000)
    ap.add_argument("--new-tokens", type=int, default=1000)
    ap.add_argument("--scheduler-steps", type=int, default=16)
    ap.add_argument("--prefix-caching", action="store_true")
    ap.add_argument("--http", type=int, default=0, help="drive the completion server over HTTP with this many concurrent requests")
    ap.add_argument("--stream", action="store_true")
    a = ap.parse_args()
    if a.http:
        import asyncio

        print(json.dumps(asyncio.run(run_http(a.http, a.prompt_len, a.new_tokens, a.stream, a.scheduler_steps, a.seqs))))
        return
    print(json.dumps(run(a.seqs, a.prompt_len, a.new_tokens, a.scheduler_steps, a.prefix_caching)))


if __name__ == "__main__":
    main()
