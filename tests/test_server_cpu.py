"""OpenAI protocol conformance of the completion server (CPU, reference runner, in-process ASGI)."""
import asyncio
import json

import httpx
import pytest

from art_b200.engine.engine import Engine
from art_b200.engine.kv_cache import BlockManager
from art_b200.engine.runner import ReferenceRunner
from art_b200.engine.server import OpenAIServer
from art_b200.engine.tool_parser import HermesToolParser
from art_b200.local.tokenizer import ByteChatTokenizer
from art_b200.models.config import PRESETS
from art_b200.models.weights import LoraConfig, init_base_weights, init_lora


@pytest.fixture(scope="module")
def server():
    cfg = PRESETS["tiny"]
    base = init_base_weights(cfg, seed=0)
    tok = ByteChatTokenizer(cfg.vocab_size)
    eng = Engine(ReferenceRunner(cfg, base, LoraConfig(), max_loras=2), BlockManager(256, 4, True),
                 eos_token_id=tok.eos_token_id, max_loras=2, num_scheduler_steps=2, max_model_len=512)
    eng.set_adapter("agent-001", init_lora(cfg, LoraConfig()))
    eng.start()
    srv = OpenAIServer(eng, tok, "tiny-base")
    yield srv
    eng.shutdown()


def client(srv):
    return httpx.AsyncClient(transport=httpx.ASGITransport(app=srv.app), base_url="http://t",
                             headers={"Authorization": "Bearer default"})


def test_models_and_auth(server):
    async def main():
        async with client(server) as c:
            r = await c.get("/v1/models")
            assert [m["id"] for m in r.json()["data"]] == ["tiny-base", "agent-001"]
            r = await c.get("/v1/models", headers={"Authorization": "Bearer nope"})
            assert r.status_code == 401
            r = await c.post("/v1/chat/completions", json={"model": "ghost", "messages": [{"role": "user", "content": "x"}]})
            assert r.status_code == 404
    asyncio.run(main())


def test_chat_completion_always_has_token_id_logprobs(server):
    async def main():
        async with client(server) as c:
            body = {"model": "agent-001", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 5, "n": 2, "seed": 1}
            r = await c.post("/v1/chat/completions", json=body)
            assert r.status_code == 200
            d = r.json()
            assert len(d["choices"]) == 2 and d["usage"]["completion_tokens"] == 10
            for ch in d["choices"]:
                lps = ch["logprobs"]["content"]
                assert len(lps) == 5 and all(e["token"].startswith("token_id:") and e["logprob"] <= 0 for e in lps)
                assert ch["finish_reason"] in ("length", "stop")
            from openai.types.chat import ChatCompletion
            ChatCompletion.model_validate(d)            # parses as the official type
    asyncio.run(main())


def test_streaming_with_usage_folds_back(server):
    from openai.types.chat.chat_completion_chunk import ChatCompletionChunk

    from art_b200.openai import consume_chat_completion_stream

    async def main():
        async with client(server) as c:
            body = {"model": "tiny-base", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 4, "stream": True,
                    "stream_options": {"include_usage": True}, "temperature": 0}
            chunks = []
            async with c.stream("POST", "/v1/chat/completions", json=body) as r:
                async for line in r.aiter_lines():
                    if line.startswith("data: ") and line != "data: [DONE]":
                        chunks.append(ChatCompletionChunk.model_validate(json.loads(line[6:])))

            class S:
                def __aiter__(self):
                    async def g():
                        for ch in chunks:
                            yield ch
                    return g()

            comp = await consume_chat_completion_stream(S())
            assert len(comp.choices[0].logprobs.content) == 4
            assert comp.usage.completion_tokens == 4 and comp.usage.prompt_tokens > 0
            # non-streaming greedy gives the same tokens
            body2 = {k: v for k, v in body.items() if k not in ("stream", "stream_options")}
            full = (await c.post("/v1/chat/completions", json=body2)).json()
            assert [e["token"] for e in full["choices"][0]["logprobs"]["content"]] == \
                [e.token for e in comp.choices[0].logprobs.content]
    asyncio.run(main())


def test_guided_choice_and_completions(server):
    async def main():
        async with client(server) as c:
            body = {"model": "tiny-base", "messages": [{"role": "user", "content": "pick"}], "guided_choice": ["yes", "no"],
                    "temperature": 0}
            d = (await c.post("/v1/chat/completions", json=body)).json()
            assert d["choices"][0]["message"]["content"] in ("yes", "no")
            assert len(d["choices"][0]["logprobs"]["content"]) == len(d["choices"][0]["message"]["content"]) + 1
            r = await c.post("/v1/completions", json={"model": "tiny-base", "prompt": "abc", "max_tokens": 3})
            assert len(r.json()["choices"][0]["logprobs"]["tokens"]) == 3
            r = await c.post("/tokenize", json={"prompt": "abc"})
            assert r.json()["tokens"] == [97, 98, 99]
    asyncio.run(main())


def test_hermes_tool_parser():
    p = HermesToolParser()
    text = 'Let me check.\n<tool_call>\n{"name": "search", "arguments": {"q": "x"}}\n</tool_call>'
    content, calls = p.extract(text)
    assert content == "Let me check.\n" and calls[0]["function"]["name"] == "search"      # kept as written
    assert json.loads(calls[0]["function"]["arguments"]) == {"q": "x"}
    assert p.extract("no tools here") == ("no tools here", [])
    assert p.extract("<tool_call>not json</tool_call>")[1] == []


def test_top_logprobs_penalties_and_logit_bias(server):
    async def main():
        async with client(server) as c:
            msgs = [{"role": "user", "content": "hello there"}]
            base = {"model": "tiny-base", "messages": msgs, "max_tokens": 6, "temperature": 0.0}
            plain = (await c.post("/v1/chat/completions", json=base)).json()["choices"][0]["logprobs"]["content"]
            assert all(e["top_logprobs"] == [] for e in plain)
            # top_logprobs: k alternatives per token, most likely first; the greedy token is alternative 0
            r = await c.post("/v1/chat/completions", json={**base, "logprobs": True, "top_logprobs": 3})
            d = r.json()
            from openai.types.chat import ChatCompletion
            ChatCompletion.model_validate(d)
            content = d["choices"][0]["logprobs"]["content"]
            assert [e["token"] for e in content] == [e["token"] for e in plain]
            for e in content:
                tops = e["top_logprobs"]
                assert len(tops) == 3 and tops[0]["token"] == e["token"] and abs(tops[0]["logprob"] - e["logprob"]) < 1e-4
                assert tops[0]["logprob"] >= tops[1]["logprob"] >= tops[2]["logprob"]
            # a large positive bias forces that token; a large negative bias on the greedy tokens bans them
            forced = (await c.post("/v1/chat/completions", json={**base, "logit_bias": {"77": 100}})).json()
            assert [e["token"] for e in forced["choices"][0]["logprobs"]["content"]] == ["token_id:77"] * 6
            banned_ids = {int(e["token"].split(":")[1]) for e in plain}
            banned = (await c.post("/v1/chat/completions", json={**base, "logit_bias": {str(t): -100 for t in banned_ids}})).json()
            assert not banned_ids & {int(e["token"].split(":")[1]) for e in banned["choices"][0]["logprobs"]["content"]}
            # frequency / presence / repetition penalties: after a strong bias towards two tokens, penalties stop the
            # repetition that the bias alone would cause
            two = {"77": 30, "78": 29.5}
            rep = (await c.post("/v1/chat/completions", json={**base, "logit_bias": two})).json()
            assert {e["token"] for e in rep["choices"][0]["logprobs"]["content"]} == {"token_id:77"}
            for pen in ({"frequency_penalty": 2.0}, {"presence_penalty": 2.0}):
                alt = (await c.post("/v1/chat/completions", json={**base, "logit_bias": two, **pen})).json()
                toks = [e["token"] for e in alt["choices"][0]["logprobs"]["content"]]
                assert toks[0] == "token_id:77" and "token_id:78" in toks[:3]
            r = await c.post("/v1/chat/completions", json={**base, "repetition_penalty": 1.5})
            assert r.status_code == 200 and len(r.json()["choices"][0]["logprobs"]["content"]) == 6
            # bad values are 400s
            assert (await c.post("/v1/chat/completions", json={**base, "top_logprobs": 50})).status_code == 400
            assert (await c.post("/v1/chat/completions", json={**base, "logit_bias": {"x": 1}})).status_code == 400
            # the legacy completions route reports alternatives as a mapping per token
            r = await c.post("/v1/completions", json={"model": "tiny-base", "prompt": "abc", "max_tokens": 3, "logprobs": 2,
                                                      "temperature": 0.0})
            lp = r.json()["choices"][0]["logprobs"]
            assert len(lp["top_logprobs"]) == 3 and all(len(m) == 2 for m in lp["top_logprobs"])
    asyncio.run(main())


def test_http_load_benchmark_runs_against_the_server(tmp_path):
    """The load script of ``engine/bench_serving.py`` end to end on the tiny CPU model: a handful of concurrent requests
    through LocalBackend + the OpenAI client, streamed and not, with sane accounting."""
    from art_b200.engine.bench_serving import run

    arch = dict(name="tiny", vocab_size=1024, hidden_size=128, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=32,
                intermediate_size=384)
    for stream in (False, True):
        res = asyncio.run(run("random:tiny", arch, concurrency=6, iterations=2, prompt_repeats=None if stream else 3,
                              prompt_tokens=120, max_tokens=5, stream=stream, path=str(tmp_path / f"s{int(stream)}"),
                              engine_args={"max_model_len": 256, "num_scheduler_steps": 2}))
        assert res["concurrency"] == 6 and res["iterations"] == 2
        assert 4.0 < res["avg_completion_tokens"] <= 5.0 and res["avg_prompt_tokens"] > 20    # a sampled EOS ends early
        assert res["requests_per_s"] > 0 and res["completion_tokens_per_s"] > 0
        assert res["request_s"]["max"] <= res["iteration_s"]["max"] + 1e-3
        assert ("ttft_s" in res) == stream
        if stream:      # the prompt was sized to the requested token count under the serving tokenizer
            assert abs(res["avg_prompt_tokens"] - 120) <= 14


def test_stop_strings_cut_the_text_like_the_reference_engine(server):
    """A request that ends on a stop string returns nothing past it (the string itself only on request), streamed or
    not; text that could be the beginning of a stop string is held back until the next tokens decide."""
    from art_b200.engine.engine import SamplingParams

    p = SamplingParams(stop=["END", "##"])
    cut = OpenAIServer._cut_at_stop
    assert cut("abc END def", p) == "abc " and cut("a##bEND", p) == "a" and cut("plain", p) == "plain"
    assert cut("abc END def", SamplingParams(stop=["END"], include_stop_str_in_output=True)) == "abc END"
    assert cut("x", None) == "x"
    held = OpenAIServer._held_back
    assert held("abc E", p) == 1 and held("abc EN", p) == 2 and held("abc #", p) == 1 and held("abc", p) == 0

    async def main():
        async with client(server) as c:
            # find a string the model really produces, then use a piece from its middle as the stop string
            body = {"model": "tiny-base", "messages": [{"role": "user", "content": "hello"}], "max_tokens": 24, "temperature": 0}
            text = (await c.post("/v1/chat/completions", json=body)).json()["choices"][0]["message"]["content"]
            if len(text) < 6:
                return
            stop = text[3:5]
            want = text[:text.find(stop)]
            r = (await c.post("/v1/chat/completions", json={**body, "stop": stop})).json()["choices"][0]
            assert r["finish_reason"] == "stop" and r["message"]["content"] == want
            r = (await c.post("/v1/chat/completions", json={**body, "stop": [stop], "include_stop_str_in_output": True})).json()
            assert r["choices"][0]["message"]["content"] == want + stop
            got = ""
            async with c.stream("POST", "/v1/chat/completions", json={**body, "stop": stop, "stream": True}) as resp:
                async for line in resp.aiter_lines():
                    if line.startswith("data: ") and line != "data: [DONE]":
                        for ch in json.loads(line[6:])["choices"]:
                            got += ch["delta"].get("content") or ""
            assert got == want
    asyncio.run(main())


@pytest.fixture()
def long_server():
    cfg = PRESETS["tiny"]
    tok = ByteChatTokenizer(cfg.vocab_size)
    eng = Engine(ReferenceRunner(cfg, init_base_weights(cfg, seed=0), LoraConfig(), max_loras=2), BlockManager(1024, 4, True),
                 eos_token_id=tok.eos_token_id, max_loras=2, num_scheduler_steps=2, max_model_len=2048)
    eng.set_adapter("agent-001", init_lora(cfg, LoraConfig()))
    eng.start()
    yield OpenAIServer(eng, tok, "tiny-base")
    eng.shutdown()


def test_named_tool_choice_with_a_frozen_schema_forces_the_call(long_server):
    server = long_server
    """The distillation path of ``get_guided_completion_params``: a teacher's tool call becomes a one-value schema plus
    a named ``tool_choice``; the student's reply is that call, teacher-forced, with its log-probs."""
    from art_b200.guided_completion import freeze_tool_schema

    tool = {"type": "function", "function": {"name": "move", "description": "", "parameters": {
        "type": "object", "properties": {"direction": {"type": "string"}, "steps": {"type": "integer"}}}}}
    frozen = freeze_tool_schema(tool, {"direction": "left", "steps": 2})

    async def main():
        async with client(server) as c:
            body = {"model": "agent-001", "messages": [{"role": "user", "content": "go"}], "tools": [frozen],
                    "tool_choice": {"type": "function", "function": {"name": "move"}}, "max_tokens": 64}
            r = await c.post("/v1/chat/completions", json=body)
            assert r.status_code == 200, r.text
            ch = r.json()["choices"][0]
            assert ch["finish_reason"] == "tool_calls"
            call = ch["message"]["tool_calls"][0]["function"]
            assert call["name"] == "move" and json.loads(call["arguments"]) == {"direction": "left", "steps": 2}
            assert len(ch["logprobs"]["content"]) > 5 and all(e["logprob"] <= 0 for e in ch["logprobs"]["content"])
            # a schema that leaves fields free is enforced by constrained decoding instead: still a call of that tool
            r = await c.post("/v1/chat/completions", json={**body, "tools": [tool], "max_tokens": 200, "seed": 0})
            call = r.json()["choices"][0]["message"]["tool_calls"][0]["function"]
            assert call["name"] == "move" and set(json.loads(call["arguments"])) <= {"direction", "steps"}
            r = await c.post("/v1/chat/completions", json={**body, "tool_choice": {"type": "function", "function": {"name": "nope"}}})
            assert r.status_code == 400
    asyncio.run(main())


def test_health_probe_restarts_a_stopped_engine_until_the_budget_is_spent(long_server):
    srv = long_server
    eng = srv.engine
    real = eng.runner.decode
    state = {"fail": 1}

    def flaky(views, steps):
        if state["fail"] > 0:
            state["fail"] -= 1
            raise RuntimeError("injected step failure")
        return real(views, steps)

    eng.runner.decode = flaky
    eng.max_recoveries = 1

    async def main():
        body = {"model": "tiny-base", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 4}
        transport = httpx.ASGITransport(app=srv.app, raise_app_exceptions=False)
        async with httpx.AsyncClient(transport=transport, base_url="http://t",
                                     headers={"Authorization": "Bearer default"}) as c:
            r = await c.post("/v1/chat/completions", json=body)
            assert r.status_code == 500
            r = await c.get("/health")
            assert r.status_code == 200 and r.json()["status"] == "recovered" and "injected" in r.json()["after"]
            r = await c.post("/v1/chat/completions", json=body)
            assert r.status_code == 200 and r.json()["usage"]["completion_tokens"] == 4
            assert (await c.get("/metrics")).json()["recoveries"] == 1
            state["fail"] = 1
            r = await c.post("/v1/chat/completions", json=body)
            assert r.status_code == 500
            assert (await c.get("/health")).status_code == 500          # budget spent
    try:
        asyncio.run(main())
    finally:
        eng.runner.decode = real


def test_server_arguments_of_the_reference_configuration_take_effect(tmp_path):
    """CORS, root path, request ids, load tracking, response role, chat template, prefix-cache hits in ``usage``,
    request logging with ``max_log_len``, middleware by import path, TLS keywords for the listener."""
    import logging

    from art_b200.engine.server import serve_kwargs

    cfg = PRESETS["tiny"]
    tok = ByteChatTokenizer(cfg.vocab_size)
    eng = Engine(ReferenceRunner(cfg, init_base_weights(cfg, seed=0), LoraConfig(), max_loras=2), BlockManager(256, 4, True),
                 eos_token_id=tok.eos_token_id, max_loras=2, num_scheduler_steps=2, max_model_len=512)
    eng.start()
    template = tmp_path / "t.jinja"
    template.write_text("{% for m in messages %}[{{ m.role }}] {{ m.content }}\n{% endfor %}[bot] ")
    sargs = {"allowed_origins": '["https://a.example"]', "allow_credentials": True, "root_path": "/proxy",
             "enable_request_id_headers": True, "enable_server_load_tracking": True, "response_role": "bot",
             "chat_template": str(template), "enable_prompt_tokens_details": True, "max_log_len": 6,
             "middleware": ["tests.helpers_middleware.add_header"], "api_key": None,
             "ssl_keyfile": "/k.pem", "ssl_certfile": "/c.pem", "uvicorn_log_level": "info"}
    srv = OpenAIServer.from_server_args(eng, tok, "tiny-base", sargs, log_requests=True)
    assert serve_kwargs(sargs) == {"ssl_keyfile": "/k.pem", "ssl_certfile": "/c.pem", "log_level": "info"}

    records: list[str] = []

    class Grab(logging.Handler):
        def emit(self, record):
            records.append(record.getMessage())

    lg = logging.getLogger("art_b200.engine.server")
    h = Grab()
    lg.addHandler(h)
    lg.setLevel(logging.INFO)

    async def main():
        async with httpx.AsyncClient(transport=httpx.ASGITransport(app=srv.app), base_url="http://t") as c:
            r = await c.post("/tokenize", json={"messages": [{"role": "user", "content": "hello"}]})
            assert tok.decode(r.json()["tokens"]) == "[user] hello\n[bot] "
            body = {"model": "tiny-base", "messages": [{"role": "user", "content": "hello there, friend"}], "max_tokens": 3}
            r = await c.post("/v1/chat/completions", json=body, headers={"Origin": "https://a.example", "X-Request-Id": "abc"})
            assert r.status_code == 200
            assert r.headers["access-control-allow-origin"] == "https://a.example"
            assert r.headers["x-request-id"] == "abc" and r.headers["x-test-middleware"] == "1"
            d = r.json()
            assert d["choices"][0]["message"]["role"] == "bot"
            assert d["usage"]["prompt_tokens_details"] == {"cached_tokens": 0}
            r = await c.post("/v1/chat/completions", json=body)           # same prompt: served from the prefix cache
            hit = r.json()["usage"]["prompt_tokens_details"]["cached_tokens"]
            assert 0 < hit < r.json()["usage"]["prompt_tokens"] and hit % 4 == 0
            r = await c.post("/v1/chat/completions", json={**body, "stream": True, "stream_options": {"include_usage": True}})
            last = [json.loads(l[6:]) for l in r.text.splitlines() if l.startswith("data: {")][-1]
            assert last["usage"]["prompt_tokens_details"]["cached_tokens"] == hit
            assert (await c.get("/load")).json() == {"server_load": 0}
            assert "x-request-id" in (await c.get("/health")).headers
    try:
        asyncio.run(main())
    finally:
        lg.removeHandler(h)
        eng.shutdown()
    assert srv.app.root_path == "/proxy"
    logged = [m for m in records if m.startswith("request chatcmpl-")]
    assert logged and "prompt='hello '" in logged[0] and "prompt_token_ids=[91, 117, 115, 101, 114, 93]" in logged[0]


def test_reasoning_parsers_split_thinking_from_content():
    from art_b200.engine.server import split_reasoning

    q = ("<think>", "</think>", False)
    r1 = ("<think>", "</think>", True)
    assert split_reasoning("<think>a b</think>yes", q) == ("a b", "yes")
    assert split_reasoning("plain answer", q) == ("", "plain answer")
    assert split_reasoning("<think>never closed", q) == ("never closed", None)
    assert split_reasoning("a b</think>yes", r1) == ("a b", "yes")                   # the template opened the block
    assert split_reasoning("still thinking", r1) == ("still thinking", None)
    # streaming: possible tag beginnings wait
    assert split_reasoning("<thi", q, done=False) == ("", None)
    assert split_reasoning("<think>abc</th", q, done=False) == ("abc", None)
    assert split_reasoning("abc</thi", r1, done=False) == ("abc", None)
    assert split_reasoning("<think>abc</think>ye", q, done=False) == ("abc", "ye")


def test_reasoning_content_in_full_and_streamed_answers(long_server):
    """The model is made to 'think' by forcing its completion (guided choice); the server splits it."""
    eng, tok = long_server.engine, long_server.tok
    srv = OpenAIServer(eng, tok, "tiny-base", reasoning_parser="qwen3")

    async def main():
        async with client(srv) as c:
            body = {"model": "tiny-base", "messages": [{"role": "user", "content": "2+2?"}],
                    "guided_choice": ["<think>two and two</think>four"]}
            d = (await c.post("/v1/chat/completions", json=body)).json()
            msg = d["choices"][0]["message"]
            assert msg["reasoning_content"] == "two and two" and msg["content"] == "four"
            r = await c.post("/v1/chat/completions", json={**body, "stream": True})
            chunks = [json.loads(l[6:]) for l in r.text.splitlines() if l.startswith("data: {")]
            think = "".join(ch["choices"][0]["delta"].get("reasoning_content") or "" for ch in chunks if ch["choices"])
            text = "".join(ch["choices"][0]["delta"].get("content") or "" for ch in chunks if ch["choices"])
            assert think == "two and two" and text == "four"
    asyncio.run(main())


def test_structured_outputs_constrain_the_completion(long_server):
    """``guided_regex``, ``guided_json``, ``response_format`` and a tool_choice that demands a call of a tool with a
    free schema: a random-weight model produces text that satisfies the constraint, with a log-prob per token."""
    import re

    srv = long_server
    schema = {"type": "object", "properties": {"city": {"type": "string", "maxLength": 12}, "days": {"type": "integer", "minimum": 0, "maximum": 999},
                                               "units": {"enum": ["C", "F"]}}, "required": ["city", "days"]}
    tools = [{"type": "function", "function": {"name": "forecast", "parameters": schema}}]
    msgs = [{"role": "user", "content": "weather?"}]

    async def main():
        async with client(srv) as c:
            async def ask(**kw):
                r = await c.post("/v1/chat/completions", json={"model": "tiny-base", "messages": msgs, "max_tokens": 120,
                                                               "seed": 3, **kw})
                assert r.status_code == 200, r.text
                return r.json()["choices"][0]

            ch = await ask(guided_regex=r"(yes|no|maybe)[.!]")
            assert re.fullmatch(r"(yes|no|maybe)[.!]", ch["message"]["content"]) and ch["finish_reason"] == "stop"
            assert len(ch["logprobs"]["content"]) == len(ch["message"]["content"])          # byte tokenizer: one per character
            ch = await ask(guided_json=schema)
            val = json.loads(ch["message"]["content"])
            assert isinstance(val["city"], str) and len(val["city"]) <= 12 and isinstance(val["days"], int)
            assert val.get("units", "C") in ("C", "F")
            ch = await ask(response_format={"type": "json_schema", "json_schema": {"name": "s", "schema": schema}}, temperature=0)
            assert set(json.loads(ch["message"]["content"])) >= {"city", "days"}
            ch = await ask(tools=tools, tool_choice={"type": "function", "function": {"name": "forecast"}})
            call = ch["message"]["tool_calls"][0]["function"]
            assert call["name"] == "forecast" and isinstance(json.loads(call["arguments"])["days"], int)
            assert ch["finish_reason"] == "tool_calls"
            ch = await ask(tools=tools, tool_choice="required", stream=False)
            assert ch["message"]["tool_calls"][0]["function"]["name"] == "forecast"
            # streamed, two choices
            r = await c.post("/v1/chat/completions", json={"model": "tiny-base", "messages": msgs, "max_tokens": 40, "n": 2,
                                                           "guided_regex": r"[0-9]{3}-[0-9]{4}", "stream": True})
            text = {0: "", 1: ""}
            for line in r.text.splitlines():
                if line.startswith("data: {"):
                    for chs in json.loads(line[6:])["choices"]:
                        text[chs["index"]] += chs["delta"].get("content") or ""
            assert all(re.fullmatch(r"[0-9]{3}-[0-9]{4}", t) for t in text.values())
            # /v1/completions takes the same fields; bad constraints are the caller's error
            r = await c.post("/v1/completions", json={"model": "tiny-base", "prompt": "n=", "max_tokens": 10, "guided_regex": r"-?[1-9][0-9]?"})
            assert re.fullmatch(r"-?[1-9][0-9]?", r.json()["choices"][0]["text"])
            r = await c.post("/v1/chat/completions", json={"model": "tiny-base", "messages": msgs, "guided_regex": "(unclosed"})
            assert r.status_code == 400 and "structured-output" in r.text
            r = await c.post("/v1/chat/completions", json={"model": "tiny-base", "messages": msgs, "guided_grammar": "root ::= x"})
            assert r.status_code == 400
    asyncio.run(main())


def test_text_completions_batch_echo_and_stream(server):
    """``/v1/completions`` with a list of prompts, ``echo`` (prompt text and prompt log-probs in front) and streaming."""
    async def main():
        async with client(server) as c:
            r = await c.post("/v1/completions", json={"model": "tiny-base", "prompt": ["ab", [104, 105, 33]], "max_tokens": 3, "n": 2,
                                                      "temperature": 0, "logprobs": 1})
            d = r.json()
            assert r.status_code == 200 and [ch["index"] for ch in d["choices"]] == [0, 1, 2, 3]
            assert d["choices"][0]["text"] == d["choices"][1]["text"] and d["usage"]["prompt_tokens"] == 5
            assert d["usage"]["completion_tokens"] == 12 and len(d["choices"][2]["logprobs"]["top_logprobs"]) == 3
            plain = d["choices"][2]
            r = await c.post("/v1/completions", json={"model": "tiny-base", "prompt": [104, 105, 33], "max_tokens": 3,
                                                      "temperature": 0, "echo": True})
            e = r.json()["choices"][0]
            assert e["text"] == "hi!" + plain["text"]
            assert e["logprobs"]["tokens"][:3] == ["token_id:104", "token_id:105", "token_id:33"]
            lps = e["logprobs"]["token_logprobs"]
            assert lps[0] is None and all(x <= 0 for x in lps[1:]) and len(lps) == 6
            assert lps[3:] == pytest.approx(plain["logprobs"]["token_logprobs"], abs=1e-4)
            r = await c.post("/v1/completions", json={"model": "tiny-base", "prompt": ["hi!", "ab"], "max_tokens": 3, "temperature": 0,
                                                      "stream": True, "stream_options": {"include_usage": True}})
            chunks = [json.loads(l[6:]) for l in r.text.splitlines() if l.startswith("data: {")]
            assert r.text.rstrip().endswith("data: [DONE]")
            text = {0: "", 1: ""}
            for ch in chunks:
                for x in ch["choices"]:
                    text[x["index"]] += x["text"]
            assert text[0] == plain["text"] and chunks[-1]["usage"]["completion_tokens"] == 6
            fins = [x["finish_reason"] for ch in chunks for x in ch["choices"] if x["finish_reason"]]
            assert fins == ["length", "length"]
            r = await c.post("/v1/completions", json={"model": "tiny-base", "prompt": [], "max_tokens": 3})
            assert r.status_code == 400
    asyncio.run(main())


def test_min_tokens_allowed_ids_bad_words_and_open_final_message(server):
    tok = server.tok

    async def main():
        async with client(server) as c:
            base = {"model": "tiny-base", "messages": [{"role": "user", "content": "hi"}], "seed": 11}
            # only the digits may be drawn
            digits = [ord(ch) for ch in "0123456789"]
            d = (await c.post("/v1/chat/completions", json={**base, "max_tokens": 12, "allowed_token_ids": digits})).json()
            assert re.fullmatch(r"[0-9]{12}", d["choices"][0]["message"]["content"])
            # ... digits and the end marker, which min_tokens keeps away for the first 8 tokens
            d = (await c.post("/v1/chat/completions", json={**base, "max_tokens": 30, "min_tokens": 8, "logit_bias": {str(tok.eos_token_id): 100},
                                                            "allowed_token_ids": digits + [tok.eos_token_id]})).json()
            ch = d["choices"][0]
            assert ch["finish_reason"] == "stop" and len(ch["logprobs"]["content"]) == 9 and re.fullmatch(r"[0-9]{8}", ch["message"]["content"])
            # bad words: "1" never appears, "23" never appears as a pair although 2 and 3 do
            d = (await c.post("/v1/chat/completions", json={**base, "max_tokens": 200, "allowed_token_ids": [ord(x) for x in "1234"],
                                                            "bad_words": ["1", "23"]})).json()
            text = d["choices"][0]["message"]["content"]
            assert len(text) == 200 and "1" not in text and "23" not in text and "2" in text and "3" in text and "4" in text
            # the last message stays open and is continued
            msgs = [{"role": "user", "content": "count"}, {"role": "assistant", "content": "1, 2, "}]
            r = await c.post("/tokenize", json={"messages": msgs, "continue_final_message": True})
            assert tok.decode(r.json()["tokens"]).endswith("<|im_start|>assistant\n1, 2, ")
            r = await c.post("/v1/chat/completions", json={"model": "tiny-base", "messages": msgs, "continue_final_message": True, "max_tokens": 3})
            assert r.status_code == 200
            ids = (await c.post("/tokenize", json={"prompt": "héllo"})).json()["tokens"]
            assert (await c.post("/detokenize", json={"tokens": ids})).json() == {"prompt": "héllo"}
            assert (await c.get("/version")).json()["version"] and (await c.get("/ping")).status_code == 200
    import re
    asyncio.run(main())


def test_prompt_logprobs_come_back_with_the_completion(server):
    async def main():
        async with client(server) as c:
            body = {"model": "agent-001", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 2, "prompt_logprobs": 1}
            d = (await c.post("/v1/chat/completions", json=body)).json()
            n = d["usage"]["prompt_tokens"]
            plp = d["prompt_logprobs"]
            assert len(plp) == n and plp[0] is None
            ids = (await c.post("/tokenize", json={"messages": body["messages"]})).json()["tokens"]
            for t, e in zip(ids[1:], plp[1:]):
                (k, v), = e.items()
                assert int(k) == t and v["logprob"] <= 0 and isinstance(v["decoded_token"], str)
    asyncio.run(main())


def test_incremental_decoder_equals_a_full_decode_and_waits_for_whole_characters():
    import random

    from art_b200.engine.server import IncrementalDecoder

    tok = ByteChatTokenizer(512)
    text = "héllo wörld 日本語 ✓ done"
    ids = tok.encode(text)
    dec = IncrementalDecoder(tok)
    pieces = [dec.push(t) for t in ids]
    assert "".join(pieces) == text == dec.text == dec.final()
    assert "" in pieces and all("�" not in p for p in pieces)         # bytes inside a character emit nothing yet
    # a completion cut in the middle of a character: final() still returns what a full decode returns
    cut = ids[: ids.index("日".encode()[0]) + 2]
    dec = IncrementalDecoder(tok)
    for t in cut:
        dec.push(t)
    assert dec.final() == tok.decode(cut, skip_special_tokens=True) and dec.text == "héllo wörld "
    # random byte soup, specials included
    rng = random.Random(0)
    for _ in range(50):
        ids = [rng.choice([rng.randrange(32, 127), rng.randrange(0xC3, 0xC5), rng.randrange(0x80, 0xC0), 256, 257]) for _ in range(40)]
        dec = IncrementalDecoder(tok)
        for t in ids:
            dec.push(t)
        assert dec.final() == tok.decode(ids, skip_special_tokens=True)


def test_stream_chunks_carry_a_scheduler_step_each_or_one_token_on_request(server):
    """The fixture's engine takes two decode steps per scheduler iteration: a stream then has two tokens per chunk;
    ``stream_per_token`` restores one chunk per token.  Both fold back into the same completion."""
    from art_b200.openai import consume_chat_completion_stream
    from openai.types.chat.chat_completion_chunk import ChatCompletionChunk

    per_token = OpenAIServer(server.engine, server.tok, "tiny-base", stream_per_token=True)
    body = {"model": "tiny-base", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 8, "stream": True,
            "temperature": 0, "ignore_eos": True}

    async def run(srv):
        async with client(srv) as c:
            r = await c.post("/v1/chat/completions", json=body)
            chunks = [ChatCompletionChunk.model_validate_json(l[6:]) for l in r.text.splitlines() if l.startswith("data: {")]
            sizes = [len(ch.choices[0].logprobs.content) for ch in chunks if ch.choices and ch.choices[0].logprobs]

            async def replay():
                for ch in chunks:
                    yield ch
            return sizes, await consume_chat_completion_stream(replay())

    (a_sizes, a), (b_sizes, b) = asyncio.run(run(server)), asyncio.run(run(per_token))
    assert sum(a_sizes) == sum(b_sizes) == 8 and max(a_sizes) == 2 and b_sizes == [1] * 8
    assert a.choices[0].message.content == b.choices[0].message.content
    assert [t.token for t in a.choices[0].logprobs.content] == [t.token for t in b.choices[0].logprobs.content]


def test_adapters_can_be_loaded_and_unloaded_while_serving(server, tmp_path):
    """The runtime adapter endpoints: a directory in PEFT layout becomes a served model name; unloading frees it."""
    from art_b200.models.peft_io import save_adapter

    cfg = PRESETS["tiny"]
    lcfg = LoraConfig()
    lora = init_lora(cfg, lcfg, seed=9)
    import torch
    g = torch.Generator().manual_seed(1)
    for k in lora:
        if "lora_B" in k:
            lora[k] = torch.randn(lora[k].shape, generator=g) * 0.3
    path = str(tmp_path / "extra")
    save_adapter(path, lora, lcfg, "tiny-base")

    async def main():
        async with client(server) as c:
            body = {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 4, "temperature": 0}
            r = await c.post("/v1/chat/completions", json={**body, "model": "extra"})
            assert r.status_code == 404
            r = await c.post("/v1/load_lora_adapter", json={"lora_name": "extra", "lora_path": path})
            assert r.status_code == 200, r.text
            assert "extra" in [m["id"] for m in (await c.get("/v1/models")).json()["data"]]
            a = (await c.post("/v1/chat/completions", json={**body, "model": "extra"})).json()["choices"][0]
            b = (await c.post("/v1/chat/completions", json={**body, "model": "tiny-base"})).json()["choices"][0]
            assert [e["logprob"] for e in a["logprobs"]["content"]] != [e["logprob"] for e in b["logprobs"]["content"]]
            assert (await c.post("/v1/load_lora_adapter", json={"lora_name": "x", "lora_path": str(tmp_path / "nope")})).status_code == 404
            assert (await c.post("/v1/unload_lora_adapter", json={"lora_name": "extra"})).status_code == 200
            assert (await c.post("/v1/chat/completions", json={**body, "model": "extra"})).status_code == 404
            assert (await c.post("/v1/unload_lora_adapter", json={"lora_name": "extra"})).status_code == 404
    asyncio.run(main())


def test_unsupported_search_modes_are_refused_not_ignored(server):
    async def main():
        async with client(server) as c:
            body = {"model": "tiny-base", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 2}
            assert (await c.post("/v1/chat/completions", json={**body, "use_beam_search": True})).status_code == 400
            assert (await c.post("/v1/chat/completions", json={**body, "n": 2, "best_of": 4})).status_code == 400
            assert (await c.post("/v1/chat/completions", json={**body, "n": 2, "best_of": 2})).status_code == 200
            # no max_tokens: the rest of the context may be used (the tiny model stops at its context of 512)
            r = await c.post("/v1/chat/completions", json={"model": "tiny-base", "messages": body["messages"], "ignore_eos": True})
            u = r.json()["usage"]
            assert u["prompt_tokens"] + u["completion_tokens"] >= 510 and r.json()["choices"][0]["finish_reason"] == "length"
    asyncio.run(main())


def test_special_tokens_can_be_kept_in_the_returned_text(server):
    tok = server.tok

    async def main():
        async with client(server) as c:
            body = {"model": "tiny-base", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 6,
                    "allowed_token_ids": [tok.IM_START, ord("a")], "seed": 4, "temperature": 1.0}
            plain = (await c.post("/v1/chat/completions", json=body)).json()["choices"][0]
            kept = (await c.post("/v1/chat/completions", json={**body, "skip_special_tokens": False})).json()["choices"][0]
            ids = [int(e["token"].split(":")[1]) for e in kept["logprobs"]["content"]]
            assert ids == [int(e["token"].split(":")[1]) for e in plain["logprobs"]["content"]] and tok.IM_START in ids
            assert "<|im_start|>" in kept["message"]["content"] and "<|im_start|>" not in plain["message"]["content"]
            assert kept["message"]["content"].replace("<|im_start|>", "") == plain["message"]["content"]
    asyncio.run(main())


def test_truncate_prompt_tokens_keeps_the_end_of_the_prompt(server):
    async def main():
        async with client(server) as c:
            long = "x" * 700                                  # more than the context of 512
            body = {"model": "tiny-base", "messages": [{"role": "user", "content": long}], "max_tokens": 2}
            assert (await c.post("/v1/chat/completions", json=body)).status_code == 400
            r = await c.post("/v1/chat/completions", json={**body, "truncate_prompt_tokens": 100})
            assert r.status_code == 200 and r.json()["usage"]["prompt_tokens"] == 100
            r = await c.post("/v1/completions", json={"model": "tiny-base", "prompt": long, "max_tokens": 2, "truncate_prompt_tokens": 64})
            assert r.json()["usage"]["prompt_tokens"] == 64
    asyncio.run(main())


def test_adapter_loading_reaches_every_replica_behind_the_leader(tmp_path):
    import socket

    import torch

    from art_b200.engine.server import serve
    from art_b200.models.peft_io import save_adapter

    cfg = PRESETS["tiny"]
    base = init_base_weights(cfg, seed=0)
    tok = ByteChatTokenizer(cfg.vocab_size)
    lcfg = LoraConfig()
    path = str(tmp_path / "extra")
    save_adapter(path, init_lora(cfg, lcfg, seed=9), lcfg, "tiny-base")

    def engine():
        e = Engine(ReferenceRunner(cfg, base, lcfg, max_loras=2), BlockManager(128, 4, True), eos_token_id=tok.eos_token_id,
                   max_loras=2, num_scheduler_steps=2, max_model_len=256)
        e.start()
        return e

    def free_port():
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            return s.getsockname()[1]

    async def main():
        e0, e1 = engine(), engine()
        p0, p1 = free_port(), free_port()
        follower = OpenAIServer(e1, tok, "tiny-base")
        leader = OpenAIServer(e0, tok, "tiny-base", peers=[f"http://127.0.0.1:{p1}"])
        r0, r1 = asyncio.Event(), asyncio.Event()
        tasks = [asyncio.create_task(serve(leader, "127.0.0.1", p0, ready=r0)), asyncio.create_task(serve(follower, "127.0.0.1", p1, ready=r1))]
        await r0.wait()
        await r1.wait()
        try:
            async with httpx.AsyncClient(headers={"Authorization": "Bearer default"}, timeout=60) as c:
                r = await c.post(f"http://127.0.0.1:{p0}/v1/load_lora_adapter", json={"lora_name": "extra", "lora_path": path})
                assert r.status_code == 200, r.text
                assert "extra" in e0.adapters and "extra" in e1.adapters
                for _ in range(4):      # wherever the leader routes it, the name is known
                    r = await c.post(f"http://127.0.0.1:{p0}/v1/chat/completions",
                                     json={"model": "extra", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 2})
                    assert r.status_code == 200, r.text
                r = await c.post(f"http://127.0.0.1:{p0}/v1/unload_lora_adapter", json={"lora_name": "extra"})
                assert r.status_code == 200 and "extra" not in e0.adapters and "extra" not in e1.adapters
        finally:
            for t in tasks:
                t.cancel()
            await asyncio.gather(*tasks, return_exceptions=True)
            e0.shutdown()
            e1.shutdown()
    asyncio.run(main())


def test_prometheus_metrics_parse(server):
    from prometheus_client.parser import text_string_to_metric_families

    async def main():
        async with client(server) as c:
            await c.post("/v1/chat/completions", json={"model": "tiny-base", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 3})
            r = await c.get("/metrics/prometheus")
            assert r.status_code == 200 and r.headers["content-type"].startswith("text/plain")
            fams = {f.name: f for f in text_string_to_metric_families(r.text)}
            assert fams["art_b200_generated_tokens"].type == "counter" and fams["art_b200_generated_tokens"].samples[0].value >= 3
            assert fams["art_b200_kv_free_blocks"].type == "gauge" and "art_b200_requests_in_flight" in fams
    asyncio.run(main())


def test_served_model_names_and_the_logprob_limit(server):
    srv = OpenAIServer(server.engine, server.tok, "tiny-base", extra_base_names=["alias-a", "tiny-base"], max_logprobs=3)

    async def main():
        async with client(srv) as c:
            ids = [m["id"] for m in (await c.get("/v1/models")).json()["data"]]
            assert ids[:2] == ["tiny-base", "alias-a"]
            body = {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 2, "temperature": 0}
            a = (await c.post("/v1/chat/completions", json={**body, "model": "alias-a"})).json()["choices"][0]["message"]["content"]
            b = (await c.post("/v1/chat/completions", json={**body, "model": "tiny-base"})).json()["choices"][0]["message"]["content"]
            assert a == b
            assert (await c.post("/v1/chat/completions", json={**body, "model": "tiny-base", "logprobs": True, "top_logprobs": 4})).status_code == 400
            assert (await c.post("/v1/chat/completions", json={**body, "model": "tiny-base", "logprobs": True, "top_logprobs": 3})).status_code == 200
    asyncio.run(main())
