"""HTTP load benchmark of the completion server: ``python -m art_b200.engine.bench_serving --model qwen2.5-7b``.

Registers a trainable model with a ``LocalBackend`` (so the numbers include everything a rollout pays: the OpenAI
client, HTTP, chat templating, the scheduler, detokenisation, log-prob reporting), then sends ``--concurrency``
chat-completion requests at once, ``--iterations`` times, and reports wall time per iteration, request latency
statistics, prompt / completion token counts and tokens per second.

Parity: the reference's load script ``dev/new_models/benchmark_inference.py:36-119`` (800 concurrent requests of about
1000 prompt tokens asking for 1000 completion tokens, Qwen2.5-14B); the same defaults are used here, with a
random-weight model of the named architecture when no local checkpoint directory is given.
"""
from __future__ import annotations

import argparse
import asyncio
import json
import statistics
import tempfile
import time


async def timed_request(client, model_name: str, prompt: str, max_tokens: int, temperature: float, stream: bool) -> dict:
    """One chat completion; returns elapsed seconds, time to the first token (streaming only) and token usage."""
    t0 = time.perf_counter()
    first = None
    if stream:
        n_out, usage = 0, None
        resp = await client.chat.completions.create(model=model_name, messages=[{"role": "user", "content": prompt}],
                                                    max_tokens=max_tokens, temperature=temperature, stream=True,
                                                    stream_options={"include_usage": True})
        async for chunk in resp:
            if chunk.choices and chunk.choices[0].logprobs and chunk.choices[0].logprobs.content:
                if first is None:
                    first = time.perf_counter() - t0
                n_out += len(chunk.choices[0].logprobs.content)
            if getattr(chunk, "usage", None):
                usage = chunk.usage
        return {"elapsed": time.perf_counter() - t0, "ttft": first,
                "prompt_tokens": usage.prompt_tokens if usage else None,
                "completion_tokens": usage.completion_tokens if usage else n_out}
    resp = await client.chat.completions.create(model=model_name, messages=[{"role": "user", "content": prompt}],
                                                max_tokens=max_tokens, temperature=temperature)
    u = resp.usage
    return {"elapsed": time.perf_counter() - t0, "ttft": None, "prompt_tokens": u.prompt_tokens if u else None,
            "completion_tokens": u.completion_tokens if u else None}


def _stats(xs: list[float]) -> dict:
    if not xs:
        return {}
    s = sorted(xs)
    return {"min": round(s[0], 4), "max": round(s[-1], 4), "mean": round(statistics.mean(s), 4),
            "p50": round(s[len(s) // 2], 4), "p95": round(s[min(len(s) - 1, int(0.95 * len(s)))], 4),
            "stdev": round(statistics.stdev(s), 4) if len(s) > 1 else 0.0}


async def run(base_model: str, architecture: dict | None = None, concurrency: int = 800, iterations: int = 1,
              prompt_repeats: int | None = None, prompt_tokens: int = 1000, max_tokens: int = 1000, temperature: float = 1.0, stream: bool = False,
              path: str | None = None, engine_args: dict | None = None, in_process: bool = True) -> dict:
    import art_b200 as art
    from art_b200.local import LocalBackend

    def make_prompt(reps: int) -> str:
        return ("Hello world. " * reps).strip() + "Please repeat the entire prompt back to me verbatim"

    init_args: dict = {}
    if architecture is not None:
        init_args["architecture"] = architecture
    model = art.TrainableModel(name="benchmark", project="benchmark-serving", base_model=base_model,
                               _internal_config={"init_args": init_args, "engine_args": dict(engine_args or {})})
    backend = LocalBackend(in_process=in_process, path=path or tempfile.mkdtemp(prefix="art-bench-serving-"))
    durations, results, engine_metrics = [], [], {}
    try:
        await model.register(backend)
        client = model.openai_client()
        name = model.get_inference_name()
        if prompt_repeats is None:
            # the reference's prompt is about 1000 tokens under its tokenizer; size ours to ``prompt_tokens`` under the
            # tokenizer that is actually serving (the offline byte-level tokenizer needs far fewer repetitions)
            import httpx

            async with httpx.AsyncClient(timeout=60) as hc:
                url = str(client.base_url).rstrip("/").removesuffix("/v1") + "/tokenize"
                n1 = (await hc.post(url, json={"messages": [{"role": "user", "content": make_prompt(1)}]})).json()["count"]
                n9 = (await hc.post(url, json={"messages": [{"role": "user", "content": make_prompt(9)}]})).json()["count"]
            per = max(1e-6, (n9 - n1) / 8)
            prompt_repeats = max(1, round((prompt_tokens - (n1 - per)) / per))
        prompt = make_prompt(prompt_repeats)
        await timed_request(client, name, "warm up", 4, temperature, stream)
        for i in range(iterations):
            t0 = time.perf_counter()
            res = await asyncio.gather(*[timed_request(client, name, prompt, max_tokens, temperature, stream)
                                         for _ in range(concurrency)])
            durations.append(time.perf_counter() - t0)
            results += res
        try:      # where the engine's time went: inside the runner (device work) or in the scheduler around it
            import httpx

            async with httpx.AsyncClient(timeout=60) as hc:
                url = str(client.base_url).rstrip("/").removesuffix("/v1") + "/metrics"
                em = (await hc.get(url, params={"format": "json"})).json()
            engine_metrics = {k: em[k] for k in ("decode_steps", "prefill_steps", "runner_seconds", "step_seconds", "preemptions",
                                                 "kv_total_blocks") if k in em}
        except Exception:  # noqa: BLE001 - the metrics are a diagnostic, not the measurement
            engine_metrics = {}
        await client.close()
    finally:
        for s in getattr(backend, "_services", {}).values():
            await s.shutdown()
        backend.close()
    total = sum(durations)
    comp = sum(r["completion_tokens"] or 0 for r in results)
    prom = sum(r["prompt_tokens"] or 0 for r in results)
    out = {"op": "serving_load", "model": base_model, "concurrency": concurrency, "iterations": iterations,
           "prompt_repeats": prompt_repeats,
           "total_s": round(total, 3), "iteration_s": _stats(durations), "request_s": _stats([r["elapsed"] for r in results]),
           "requests_per_s": round(len(results) / total, 2), "avg_prompt_tokens": round(prom / max(1, len(results)), 1),
           "avg_completion_tokens": round(comp / max(1, len(results)), 1),
           "completion_tokens_per_s": round(comp / total, 1), "total_tokens_per_s": round((comp + prom) / total, 1)}
    if engine_metrics:
        out["engine"] = engine_metrics
    ttft = [r["ttft"] for r in results if r["ttft"] is not None]
    if ttft:
        out["ttft_s"] = _stats(ttft)
    return out


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--model", default="qwen2.5-7b", help="architecture preset (random weights) or a local checkpoint directory")
    ap.add_argument("--concurrency", type=int, default=800)
    ap.add_argument("--iterations", type=int, default=1)
    ap.add_argument("--prompt-repeats", type=int, default=None,
                    help='"Hello world. " repeated this often (default: as often as gives --prompt-tokens tokens)')
    ap.add_argument("--prompt-tokens", type=int, default=1000)
    ap.add_argument("--max-tokens", type=int, default=1000)
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--stream", action="store_true", help="stream the answers and report the time to the first token")
    ap.add_argument("--server-process", action="store_true",
                    help="run the model service (engine + HTTP server) in a child process, as a deployment would; "
                         "by default it shares this process, and its interpreter lock, with the 800 client coroutines")
    ap.add_argument("--max-num-seqs", type=int, default=512)
    ap.add_argument("--max-model-len", type=int, default=8192)
    a = ap.parse_args()
    import os

    base = a.model if os.path.isdir(a.model) else f"random:{a.model}"
    res = asyncio.run(run(base, None, a.concurrency, a.iterations, a.prompt_repeats, a.prompt_tokens, a.max_tokens,
                          a.temperature, a.stream,
                          engine_args={"max_num_seqs": a.max_num_seqs, "max_model_len": a.max_model_len},
                          in_process=not a.server_process))
    print(json.dumps(res))


if __name__ == "__main__":
    main()
