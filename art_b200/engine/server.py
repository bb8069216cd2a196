"""OpenAI-compatible completion server in front of :class:`engine.Engine`.

Routes: ``GET /health``, ``GET /v1/models``, ``POST /v1/chat/completions`` (streaming and
non-streaming, ``n``, ``stream_options.include_usage``, tools with Hermes-format parsing and
auto tool choice, ``guided_choice``, ``chat_template_kwargs``), ``POST /v1/completions``,
``POST /tokenize``, ``GET /metrics``.

Contract details the trainer depends on (reference: ``src/art/dev/openai_server.py:7-35`` and the
request subclass at ``src/art/local/vllm.py:234-247``):

* log-probs are **always** returned (``top_logprobs`` defaults to 0), and every sampled token is
  reported, including the tokens of tool calls;
* with ``return_tokens_as_token_ids`` (default on) token strings are ``token_id:{id}`` so the
  tokenizer pipeline can splice the exact sampled ids back into the conversation;
* the ``model`` field routes by name: a registered adapter name selects that LoRA, the base
  model name selects no adapter;
* a client that disconnects mid-stream aborts its request and nothing else.
"""
from __future__ import annotations

import asyncio
import importlib
import logging
import os
import json
import time
import uuid
from collections.abc import Mapping
from typing import Any, AsyncIterator

from fastapi import FastAPI, HTTPException, Request
from fastapi.responses import JSONResponse, StreamingResponse

from .engine import Engine, SamplingParams
from .tool_parser import HermesToolParser


_log = logging.getLogger(__name__)


def _now() -> int:
    return int(time.time())


# reasoning parsers: name -> (opening tag, closing tag, block open from the start).  The last is True for model
# families whose chat template opens the block itself, so that a completion starts inside it without an opening tag.
_REASONING_TAGS = {"deepseek_r1": ("<think>", "</think>", True), "qwen3": ("<think>", "</think>", False),
                   "granite": ("<think>", "</think>", False)}


def _load_template(spec: str | None) -> str | None:
    """A chat template given as a file path or as the template text itself."""
    if not spec:
        return None
    if "{" not in spec and os.path.exists(spec):
        with open(spec) as f:
            return f.read()
    return spec


def split_reasoning(text: str, tags: tuple[str, str, bool], done: bool = True) -> tuple[str, str | None]:
    """``(reasoning, content)`` of a completion.  With a closing tag, what precedes it is the reasoning (an opening
    tag at its start is dropped) and what follows is the content.  With an opening tag only, or with neither tag
    when the parser's block is open from the start, everything is reasoning and the content is None.  Otherwise the
    text is content.  ``done`` False is the streaming case: a trailing piece that may still become the closing tag is
    held back, and a text that may still become the opening tag is neither yet."""
    open_t, close_t, implicit = tags
    if close_t in text:
        r, _, c = text.partition(close_t)
        r = r.lstrip()
        return (r[len(open_t):] if r.startswith(open_t) else r), c
    lead = text.lstrip()
    if lead.startswith(open_t):
        body = lead[len(open_t):]
        return (body if done else _without_partial(body, close_t)), None
    if not done and lead and open_t.startswith(lead):
        return "", None
    if implicit:
        return (text if done else _without_partial(text, close_t)), None
    return "", text


def _without_partial(text: str, tag: str) -> str:
    """``text`` without a trailing proper prefix of ``tag`` (held back while streaming)."""
    for k in range(min(len(tag) - 1, len(text)), 0, -1):
        if text.endswith(tag[:k]):
            return text[:-k]
    return text


class IncrementalDecoder:
    """Text of a growing token sequence without decoding it from the start at every token: only a short window of
    recent tokens is decoded (the part already turned into text, to have its length, and the same plus what is new),
    and nothing is emitted while the window ends in half a character.  Cost per token is constant; decoding the whole
    completion at every token made a streamed 1000-token answer cost 500 000 token decodes."""

    def __init__(self, tok, skip_special_tokens: bool = True):
        self.tok, self.skip = tok, skip_special_tokens
        self.ids: list[int] = []
        self.prefix = self.read = 0
        self.text = ""

    def push(self, tid: int) -> str:
        """Adds a token; returns the text it completed ("" while a character is still open)."""
        return self.extend((tid,))

    def extend(self, tids) -> str:
        """Adds the tokens of one step with one pass over the window."""
        self.ids.extend(tids)
        old = self.tok.decode(self.ids[self.prefix:self.read], skip_special_tokens=self.skip) if self.read > self.prefix else ""
        new = self.tok.decode(self.ids[self.prefix:], skip_special_tokens=self.skip)
        if len(new) > len(old) and not new.endswith("\ufffd"):
            delta = new[len(old):]
            self.prefix, self.read = self.read, len(self.ids)
            self.text += delta
            return delta
        return ""

    def final(self) -> str:
        """The whole text, including a trailing piece that never became a full character."""
        if self.read == len(self.ids):
            return self.text
        old = self.tok.decode(self.ids[self.prefix:self.read], skip_special_tokens=self.skip) if self.read > self.prefix else ""
        new = self.tok.decode(self.ids[self.prefix:], skip_special_tokens=self.skip)
        return self.text + new[len(old):]


class OpenAIServer:
    def __init__(self, engine: Engine, tokenizer, base_model_name: str, *, api_key: str | None = "default",
                 return_tokens_as_token_ids: bool = True, enable_auto_tool_choice: bool = True,
                 tool_call_parser: str | None = "hermes", default_max_tokens: int | None = None, peers: list[str] | None = None,
                 response_role: str | None = None, chat_template: str | None = None, root_path: str | None = None,
                 cors: dict | None = None, middleware: list[str] | None = None, request_id_headers: bool = False,
                 fastapi_docs: bool = False, max_log_len: int | None = None, log_requests: bool = False,
                 prompt_tokens_details: bool = False, reasoning_parser: str | None = None,
                 load_tracking: bool = False, stream_per_token: bool = False, max_logprobs: int = 20,
                 extra_base_names: list[str] | None = None):
        """``peers``: base URLs of further replicas of the same model (other GPUs of the node).  This server then
        spreads ``/v1/chat/completions`` and ``/v1/completions`` over itself and the peers, least loaded first,
        passing a peer's answer (JSON or event stream) through unchanged; a client only ever sees this one URL.

        The remaining keywords are the server arguments of the reference's configuration
        (src/art/dev/openai_server.py:60-125) with the meaning they have there: ``response_role`` (role of returned
        messages), ``chat_template`` (a template file or the template itself, used instead of the tokenizer's),
        ``root_path``, ``cors`` (``allow_origins`` / ``allow_methods`` / ``allow_headers`` / ``allow_credentials``),
        ``middleware`` (import paths of ASGI middleware classes or of ``async def f(request, call_next)`` functions),
        ``request_id_headers`` (``X-Request-Id`` on every response), ``fastapi_docs``, ``log_requests`` with
        ``max_log_len`` (prompt characters / ids printed per request), ``prompt_tokens_details`` (prefix-cache hits
        in ``usage``), ``reasoning_parser`` (text between ``<think>`` and ``</think>`` is returned as
        ``reasoning_content``), ``load_tracking`` (``GET /load``).  ``stream_per_token``: one stream chunk per token instead of
        one per scheduler step (``engine_args.multi_step_stream_outputs`` of the reference's engine; four times the host
        cost per streamed token)."""
        self.engine, self.tok = engine, tokenizer
        self.peers = list(peers or [])
        self._load = [0] * (1 + len(self.peers))       # requests in flight: [this replica, peer 0, peer 1, ...]
        self._rr = 0
        self._http = None
        self.base_model_name = base_model_name
        self.api_key = api_key
        self.token_ids_as_strings = return_tokens_as_token_ids
        self.auto_tools = enable_auto_tool_choice
        self.tool_parser = HermesToolParser() if tool_call_parser in ("hermes", None) else HermesToolParser()
        self.default_max_tokens = default_max_tokens
        self.role = response_role or "assistant"
        self.chat_template = _load_template(chat_template)
        self.root_path = root_path or ""
        self.cors = cors
        self.middleware = list(middleware or [])
        self.request_id_headers = request_id_headers
        self.fastapi_docs = fastapi_docs
        self.max_log_len = max_log_len
        self.log_requests = log_requests
        self.prompt_tokens_details = prompt_tokens_details
        self.reasoning = _REASONING_TAGS.get(reasoning_parser or "", None) if reasoning_parser else None
        if reasoning_parser and self.reasoning is None:
            raise ValueError(f"unknown reasoning parser {reasoning_parser!r}; known: {sorted(_REASONING_TAGS)}")
        self.load_tracking = load_tracking
        self.stream_per_token = stream_per_token
        self.max_logprobs = int(max_logprobs)                     # largest top_logprobs a request may ask for
        self.base_names = [base_model_name] + [n for n in (extra_base_names or []) if n != base_model_name]
        self._tok_fields: dict[int, tuple[str, list[int]]] = {}
        self.app = self._build()

    @classmethod
    def from_server_args(cls, engine: Engine, tokenizer, base_model_name: str, sargs: dict, *,
                         log_requests: bool = False, peers: list[str] | None = None,
                         stream_per_token: bool = False, max_logprobs: int = 20,
                         extra_base_names: list[str] | None = None) -> "OpenAIServer":
        """Builds the server from a ``ServerArgs`` dictionary (the keys that concern the HTTP listener itself, host,
        port, TLS files and log level, are read by :func:`serve_kwargs`)."""
        def jlist(key: str):
            v = sargs.get(key)
            if v is None:
                return None
            return json.loads(v) if isinstance(v, str) else list(v)

        cors = None
        if any(k in sargs for k in ("allowed_origins", "allowed_methods", "allowed_headers", "allow_credentials")):
            cors = {"allow_origins": jlist("allowed_origins") or ["*"], "allow_methods": jlist("allowed_methods") or ["*"],
                    "allow_headers": jlist("allowed_headers") or ["*"],
                    "allow_credentials": bool(sargs.get("allow_credentials", False))}
        return cls(engine, tokenizer, base_model_name, api_key=sargs.get("api_key", "default"),
                   return_tokens_as_token_ids=bool(sargs.get("return_tokens_as_token_ids", True)),
                   enable_auto_tool_choice=bool(sargs.get("enable_auto_tool_choice", True)),
                   tool_call_parser=sargs.get("tool_call_parser", "hermes"), peers=peers,
                   response_role=sargs.get("response_role"), chat_template=sargs.get("chat_template"),
                   root_path=sargs.get("root_path"), cors=cors, middleware=sargs.get("middleware"),
                   request_id_headers=bool(sargs.get("enable_request_id_headers", False)),
                   fastapi_docs=sargs.get("disable_fastapi_docs") is False,
                   max_log_len=sargs.get("max_log_len"), log_requests=log_requests,
                   prompt_tokens_details=bool(sargs.get("enable_prompt_tokens_details", False)),
                   reasoning_parser=(sargs.get("reasoning_parser") or "deepseek_r1") if sargs.get("enable_reasoning") else None,
                   load_tracking=bool(sargs.get("enable_server_load_tracking", False)), stream_per_token=stream_per_token,
                   max_logprobs=max_logprobs, extra_base_names=extra_base_names)

    # -- helpers ------------------------------------------------------------------------------------
    def _auth(self, request: Request) -> None:
        if not self.api_key:
            return
        got = request.headers.get("authorization", "")
        if got != f"Bearer {self.api_key}":
            raise HTTPException(status_code=401, detail="invalid api key")

    def _route(self, model: str | None) -> str | None:
        """Adapter name for ``model`` (None = base model)."""
        if model is None or model in self.base_names:
            return None
        if model in self.engine.adapters:
            return model
        raise HTTPException(status_code=404, detail=f"The model `{model}` does not exist.")

    # -- replica routing ----------------------------------------------------------------------------
    def _pick_replica(self) -> int:
        """Index into ``_load`` of the least-loaded replica (0 = this process); ties rotate."""
        n = len(self._load)
        best = min(range(n), key=lambda i: (self._load[i], (i - self._rr) % n))
        self._rr = (best + 1) % n
        return best

    async def _fan_out(self, path: str, body: dict, request: Request) -> None:
        """Repeats an administrative request (adapter load / unload) on every peer replica, so that whichever replica
        a later completion request is routed to knows the adapter; raises with the first peer's refusal."""
        if not self.peers or request.headers.get("x-art-routed"):
            return
        results = await asyncio.gather(*[self._forward(i + 1, path, {**body, "stream": False}, request)
                                         for i in range(len(self.peers))])
        for i, r in enumerate(results):
            if r.status_code >= 400:
                raise HTTPException(status_code=r.status_code, detail=f"replica {i + 1}: {bytes(r.body).decode(errors='replace')}")

    async def _forward(self, idx: int, path: str, body: dict, request: Request):
        """Send the request to peer ``idx - 1`` and pass its answer through."""
        import httpx

        if self._http is None:
            self._http = httpx.AsyncClient(timeout=httpx.Timeout(None, connect=10.0),
                                           limits=httpx.Limits(max_connections=None, max_keepalive_connections=256))
        url = self.peers[idx - 1] + path
        headers = {"authorization": request.headers.get("authorization", ""), "x-art-routed": "1"}
        self._load[idx] += 1
        if body.get("stream"):
            req = self._http.build_request("POST", url, json=body, headers=headers)
            try:
                resp = await self._http.send(req, stream=True)
            except BaseException:
                self._load[idx] -= 1
                raise

            async def relay():
                try:
                    async for chunk in resp.aiter_raw():
                        yield chunk
                finally:       # also reached when the client goes away: closing the upstream aborts the request there
                    await resp.aclose()
                    self._load[idx] -= 1

            return StreamingResponse(relay(), status_code=resp.status_code,
                                     media_type=resp.headers.get("content-type", "text/event-stream"))
        try:
            resp = await self._http.post(url, json=body, headers=headers)
        finally:
            self._load[idx] -= 1
        return JSONResponse(resp.json(), status_code=resp.status_code)

    def _token_str(self, tid: int) -> str:
        return self._token_fields(tid)[0]

    def _token_fields(self, tid: int) -> tuple[str, list[int]]:
        """The ``token`` string and the ``bytes`` list of a token id, computed once per id: detokenising one token costs
        microseconds with a byte-level tokenizer and tens of them with a BPE vocabulary, per token and request."""
        hit = self._tok_fields.get(tid)
        if hit is None:
            text = self.tok.decode([tid])
            hit = self._tok_fields[tid] = (f"token_id:{tid}" if self.token_ids_as_strings else text,
                                           list(text.encode("utf-8")))
        return hit

    def _logprob_entry(self, tid: int, lp: float, top=None) -> dict:
        token, raw = self._token_fields(tid)
        alts = []
        for t, l in (top or ()):
            if t >= 0:
                tt, tb = self._token_fields(t)
                alts.append({"token": tt, "logprob": l, "bytes": tb})
        return {"token": token, "logprob": lp, "bytes": raw, "top_logprobs": alts}

    def _params(self, body: dict, prompt_len: int) -> SamplingParams:
        n_req = int(body.get("n") or 1)
        if body.get("use_beam_search") or int(body.get("best_of") or n_req) != n_req:
            raise HTTPException(status_code=400, detail="beam search and best_of are not supported (sample n choices instead)")
        # without a limit in the request a completion may use the rest of the context, as with the reference's engine
        max_tokens = (body.get("max_completion_tokens") or body.get("max_tokens") or self.default_max_tokens
                      or self.engine.max_model_len)
        max_tokens = max(1, min(int(max_tokens), self.engine.max_model_len - prompt_len - 1))
        stop = body.get("stop")
        if isinstance(stop, str):
            stop = [stop]
        temp = body.get("temperature")
        top_lp = body.get("top_logprobs")
        if top_lp is None and isinstance(body.get("logprobs"), int) and not isinstance(body.get("logprobs"), bool):
            top_lp = body["logprobs"]                       # /v1/completions spelling
        top_lp = int(top_lp or 0)
        if not 0 <= top_lp <= self.max_logprobs:
            raise HTTPException(status_code=400, detail=f"top_logprobs must be between 0 and {self.max_logprobs}")
        bias = body.get("logit_bias") or None
        if bias:
            try:
                bias = {int(k): max(-100.0, min(100.0, float(v))) for k, v in bias.items()}
            except (TypeError, ValueError) as e:
                raise HTTPException(status_code=400, detail="logit_bias maps token ids to numbers") from e
        rep = float(body.get("repetition_penalty") or 1.0)
        if rep <= 0:
            raise HTTPException(status_code=400, detail="repetition_penalty must be positive")
        return SamplingParams(top_logprobs=top_lp, repetition_penalty=rep,
                              presence_penalty=float(body.get("presence_penalty") or 0.0),
                              frequency_penalty=float(body.get("frequency_penalty") or 0.0), logit_bias=bias,
                              max_tokens=max_tokens, temperature=1.0 if temp is None else float(temp),
                              top_p=float(body.get("top_p") or 1.0), top_k=int(body.get("top_k") or -1),
                              min_p=float(body.get("min_p") or 0.0),
                              n=int(body.get("n") or 1), stop=stop, stop_token_ids=body.get("stop_token_ids"),
                              seed=body.get("seed"), ignore_eos=bool(body.get("ignore_eos", False)),
                              guided_choice=body.get("guided_choice") or (body.get("structured_outputs") or {}).get("choice")
                              if not body.get("guided_regex") else None,
                              include_stop_str_in_output=bool(body.get("include_stop_str_in_output", False)),
                              skip_special_tokens=bool(body.get("skip_special_tokens", True)),
                              min_tokens=max(0, min(int(body.get("min_tokens") or 0), max_tokens)),
                              allowed_token_ids=[int(t) for t in body["allowed_token_ids"]] if body.get("allowed_token_ids") else None,
                              bad_words_ids=self._bad_words(body.get("bad_words")))

    def _bad_words(self, words) -> list[list[int]] | None:
        """Token sequences of the request's ``bad_words``: each word as it is and with a leading space (the two are
        different tokens in most vocabularies)."""
        if not words:
            return None
        out: list[list[int]] = []
        for w in words:
            for text in {str(w), " " + str(w).lstrip()}:
                ids = list(self.tok.encode(text, add_special_tokens=False))
                if ids and ids not in out:
                    out.append(ids)
        return out or None

    @staticmethod
    def _forced_tool_call(body: dict) -> str | None:
        """``tool_choice={"type": "function", "function": {"name": N}}``: the reply must be a call of tool N.  When that
        tool's parameter schema admits exactly one value per field (one-value enums / consts, which is what
        ``art.guided_completion.freeze_tool_schema`` builds for distillation), the whole call is determined and is
        returned here as Hermes-format text; the request then runs like ``guided_choice`` with that one candidate.
        A schema that leaves freedom returns None here and becomes a constraint on the decoding (:meth:`_guided_regex`)."""
        choice = body.get("tool_choice")
        if not isinstance(choice, dict) or choice.get("type") != "function":
            return None
        name = (choice.get("function") or {}).get("name")
        tool = next((t for t in body.get("tools") or [] if (t.get("function") or {}).get("name") == name), None)
        if tool is None:
            raise HTTPException(status_code=400, detail=f"tool_choice names {name!r}, which is not among the tools")
        schema = tool["function"].get("parameters") or {}
        args: dict = {}
        for key, spec in (schema.get("properties") or {}).items():
            if "const" in spec:
                args[key] = spec["const"]
            elif isinstance(spec.get("enum"), list) and len(spec["enum"]) == 1:
                args[key] = spec["enum"][0]
            else:
                return None
        return "<tool_call>\n" + json.dumps({"name": name, "arguments": args}) + "\n</tool_call>"

    @staticmethod
    def _has_constraint(body: dict) -> bool:
        """Whether the request carries any structured-output field (the common request has none and is not made to
        wait for the worker thread that compiles constraints)."""
        choice = body.get("tool_choice")
        return bool(body.get("guided_regex") or body.get("guided_json") is not None or body.get("structured_outputs")
                    or body.get("guided_grammar") or (body.get("response_format") or {}).get("type") in ("json_object", "json_schema")
                    or choice == "required" or (isinstance(choice, dict) and choice.get("type") == "function"))

    def _guided_regex(self, body: dict) -> str | None:
        """The regular expression a completion has to match, from whichever structured-output field the request uses:
        ``guided_regex``, ``guided_json``, ``response_format`` (``json_object`` / ``json_schema``), ``structured_outputs``
        (``{"regex" | "json" | "choice": ...}``), or a ``tool_choice`` that demands a call (a named function, or
        ``"required"``: Hermes-format call text whose arguments satisfy the tool's parameter schema)."""
        from .grammar import RegexError, compile_cached, escape_literal, schema_to_regex

        so = body.get("structured_outputs") or {}
        try:
            rx = body.get("guided_regex") or so.get("regex")
            schema = body.get("guided_json") if body.get("guided_json") is not None else so.get("json")
            if rx is None and schema is not None:
                rx = schema_to_regex(schema)
            if rx is None and so.get("choice"):
                rx = "(" + "|".join(escape_literal(str(c)) for c in so["choice"]) + ")"
            fmt = body.get("response_format") or {}
            if rx is None and fmt.get("type") == "json_object":
                rx = schema_to_regex({"type": "object"})
            if rx is None and fmt.get("type") == "json_schema":
                rx = schema_to_regex((fmt.get("json_schema") or {}).get("schema", True))
            choice = body.get("tool_choice")
            if rx is None and (choice == "required" or (isinstance(choice, dict) and choice.get("type") == "function")):
                tools = [t.get("function") or {} for t in body.get("tools") or []]
                if isinstance(choice, dict):
                    name = (choice.get("function") or {}).get("name")
                    tools = [t for t in tools if t.get("name") == name]
                if not tools:
                    raise HTTPException(status_code=400, detail="tool_choice demands a call but no matching tool is given")
                calls = [r'\{"name": "' + escape_literal(t["name"]) + '", "arguments": '
                         + schema_to_regex(t.get("parameters") or {"type": "object"}) + r"\}" for t in tools]
                rx = "<tool_call>\n(" + "|".join(calls) + ")\n</tool_call>"
            if body.get("guided_grammar") or so.get("grammar"):
                raise HTTPException(status_code=400, detail="context-free grammars are not supported; use a JSON schema or a regular expression")
            if rx is not None:
                if len(rx) > 200_000:
                    raise ValueError(f"the constraint expands to an expression of {len(rx)} characters (limit 200 000)")
                compile_cached(rx)             # syntax and size errors surface here, as a 400
        except (RegexError, ValueError, KeyError, TypeError) as e:
            raise HTTPException(status_code=400, detail=f"cannot build the structured-output constraint: {e}") from e
        return rx

    def _ensure_masker(self) -> None:
        """The allowed-token index of the serving tokenizer, built at the first structured-output request."""
        if self.engine.token_masker is None:
            from .grammar import vocabulary_bytes

            self.engine.set_vocabulary(vocabulary_bytes(self.tok), self.engine.eos)

    def _render_chat(self, body: dict) -> list[int]:
        tools = body.get("tools")
        if body.get("tool_choice") == "none":
            tools = None
        kwargs = dict(body.get("chat_template_kwargs") or {})
        template = body.get("chat_template") or self.chat_template
        if template:
            kwargs["chat_template"] = template
        cont = bool(body.get("continue_final_message", False))
        if cont:
            kwargs["continue_final_message"] = True
        ids = self.tok.apply_chat_template(body["messages"], tools=tools, tokenize=True,
                                           add_generation_prompt=bool(body.get("add_generation_prompt", not cont)), **kwargs)
        if isinstance(ids, Mapping):       # newer tokenizer libraries return the dictionary form by default
            ids = ids["input_ids"]
        return [int(t) for t in ids]

    async def _run_steps(self, prompt_ids: list[int], params: SamplingParams, adapter: str | None, index: int,
                         info: dict | None = None):
        """Async iterator over lists of (index, token_id, logprob, finished, finish_reason, top_logprobs) for one choice:
        one list per scheduler step, which is what a stream sends as one chunk.
        ``info["cached_tokens"]`` collects the prompt tokens that came out of the prefix cache."""
        if params.guided_choice:
            async for item in self._run_guided(prompt_ids, params, adapter, index):
                yield [item]
            return
        seq_params = SamplingParams(**{**params.__dict__, "n": 1,
                                       "seed": None if params.seed is None else params.seed + index})
        stops = params.stop or []
        dec = IncrementalDecoder(self.tok, params.skip_special_tokens) if stops else None
        longest = max((len(x) for x in stops), default=0)
        agen = self.engine.generate_steps(prompt_ids, seq_params, adapter)
        try:
            async for events in agen:
                out = []
                for ev in events:
                    if info is not None and getattr(ev, "cached_tokens", None):
                        info["cached_tokens"] = max(info.get("cached_tokens", 0), ev.cached_tokens)
                    out.append((index, ev.token_id, ev.logprob, ev.finished, ev.finish_reason, ev.top_logprobs))
                    if stops and not ev.finished:
                        # windowed decoding (whole characters only, like the text that is returned); only the end of
                        # the text can hold a new match
                        delta = dec.push(ev.token_id)
                        tail = dec.text[-(longest + len(delta)):] if delta else ""
                        if delta and any(s in tail for s in stops):
                            out.append((index, None, None, True, "stop", None))
                            yield out
                            return
                    if ev.finished:
                        break
                yield out
                if out and out[-1][3]:
                    return
        finally:
            await agen.aclose()

    async def _run_one(self, prompt_ids: list[int], params: SamplingParams, adapter: str | None, index: int,
                       info: dict | None = None):
        """:meth:`_run_steps`, one token at a time."""
        agen = self._run_steps(prompt_ids, params, adapter, index, info)
        try:
            async for items in agen:
                for item in items:
                    yield item
        finally:
            await agen.aclose()

    async def _run_guided(self, prompt_ids: list[int], params: SamplingParams, adapter: str | None, index: int):
        """``guided_choice``: the completion is one of the given strings.  Every candidate is scored
        under the model (teacher forcing), one is drawn from the renormalised distribution over
        candidates (arg-max at temperature 0), and its tokens are returned with their log-probs."""
        import math
        import random

        eos = [self.engine.eos] if self.engine.eos is not None else []
        cands = [list(self.tok.encode(c, add_special_tokens=False)) + eos for c in params.guided_choice]   # no BOS inside a completion
        scores = [await self.engine.score(prompt_ids, c, adapter) for c in cands]
        totals = [sum(s) for s in scores]
        if params.temperature <= 0 or len(cands) == 1:
            pick = max(range(len(cands)), key=lambda i: totals[i])
        else:
            mx = max(totals)
            w = [math.exp((t - mx) / params.temperature) for t in totals]
            rng = random.Random(None if params.seed is None else params.seed + index)
            pick = rng.choices(range(len(cands)), weights=w)[0]
        ids, lps = cands[pick], scores[pick]
        for k, (t, lp) in enumerate(zip(ids, lps)):
            last = k == len(ids) - 1
            yield index, t, lp, last, "stop" if last else None, None

    # -- app ----------------------------------------------------------------------------------------
    def _build(self) -> FastAPI:
        docs = {} if self.fastapi_docs else {"docs_url": None, "redoc_url": None, "openapi_url": None}
        app = FastAPI(title="art-b200 completion server", root_path=self.root_path, **docs)
        srv = self
        if self.cors is not None:
            from fastapi.middleware.cors import CORSMiddleware

            app.add_middleware(CORSMiddleware, **self.cors)
        for path in self.middleware:
            mod, _, attr = path.rpartition(".")
            obj = getattr(importlib.import_module(mod), attr)
            if isinstance(obj, type):
                app.add_middleware(obj)
            elif asyncio.iscoroutinefunction(obj):
                app.middleware("http")(obj)
            else:
                raise ValueError(f"middleware {path!r} is neither a class nor an async function")
        if self.request_id_headers:
            @app.middleware("http")
            async def request_id(request: Request, call_next):
                rid = request.headers.get("x-request-id") or uuid.uuid4().hex
                response = await call_next(request)
                response.headers["X-Request-Id"] = rid
                return response

        if self.load_tracking:
            @app.get("/load")
            async def load():
                return {"server_load": srv._load[0]}

        @app.get("/health")
        async def health():
            eng = srv.engine
            if eng.error is not None:
                # a health probe restarts a stopped engine while its restart budget lasts; past it the probe fails and
                # whoever supervises the server replaces the process
                err = repr(eng.error)
                if eng.recoveries >= eng.max_recoveries or not await asyncio.to_thread(eng.recover):
                    raise HTTPException(status_code=500, detail=err)
                return {"status": "recovered", "recoveries": eng.recoveries, "after": err}
            return {"status": "ok", "recoveries": eng.recoveries}

        @app.get("/metrics")
        async def metrics():
            m = srv.engine.metrics()
            if srv.peers:
                m["replica_load"] = list(srv._load)
            return m

        @app.get("/metrics/prometheus")
        async def metrics_prometheus():
            """The numeric entries of ``/metrics`` in the Prometheus text format (names prefixed ``art_b200_``; counters
            where the value only grows)."""
            from fastapi.responses import PlainTextResponse

            counters = {"prompt_tokens", "generated_tokens", "preemptions", "recoveries", "decode_steps", "prefill_steps",
                        "prefix_queries", "prefix_hits", "runner_seconds", "step_seconds"}
            lines = []
            for k, v in srv.engine.metrics().items():
                if isinstance(v, bool) or not isinstance(v, (int, float)):
                    continue
                name = f"art_b200_{k}" + ("_total" if k in counters else "")
                lines += [f"# TYPE {name} {'counter' if k in counters else 'gauge'}", f"{name} {float(v):.10g}"]
            for i, n in enumerate(srv._load):
                lines.append(f'art_b200_requests_in_flight{{replica="{i}"}} {n}')
            return PlainTextResponse("\n".join(lines) + "\n", media_type="text/plain; version=0.0.4")

        @app.get("/v1/models")
        async def models(request: Request):
            srv._auth(request)
            names = srv.base_names + list(srv.engine.adapters)
            return {"object": "list", "data": [{"id": n, "object": "model", "created": _now(), "owned_by": "art-b200",
                                                "root": srv.base_model_name,
                                                "parent": None if n in srv.base_names else srv.base_model_name}
                                               for n in names]}

        @app.get("/ping")
        async def ping():
            return await health()

        @app.get("/version")
        async def version():
            from .. import __version__

            return {"version": __version__}

        @app.post("/v1/load_lora_adapter")
        async def load_lora_adapter(request: Request):
            """Serve the adapter in the directory ``lora_path`` under the name ``lora_name`` (replacing an adapter of
            that name), between two engine steps."""
            srv._auth(request)
            body = await request.json()
            name, path = body.get("lora_name"), body.get("lora_path")
            if not name or not path:
                raise HTTPException(status_code=400, detail="lora_name and lora_path are required")
            from ..models.peft_io import is_adapter_dir, load_adapter

            if not is_adapter_dir(path):
                raise HTTPException(status_code=404, detail=f"{path} holds no adapter_model.safetensors + adapter_config.json")

            def swap():
                state, _ = load_adapter(path, getattr(srv.engine.runner, "device", "cpu"))
                srv.engine.pause()
                try:
                    srv.engine.set_adapter(name, state)
                finally:
                    srv.engine.resume()

            try:
                await asyncio.to_thread(swap)
            except (RuntimeError, ValueError, KeyError) as e:
                raise HTTPException(status_code=400, detail=f"cannot load the adapter: {e}") from e
            await srv._fan_out("/v1/load_lora_adapter", body, request)
            return {"status": "ok", "lora_name": name}

        @app.post("/v1/unload_lora_adapter")
        async def unload_lora_adapter(request: Request):
            srv._auth(request)
            name = (await request.json()).get("lora_name")
            if name not in srv.engine.adapters:
                raise HTTPException(status_code=404, detail=f"no adapter named {name!r}")

            def drop():
                srv.engine.pause()
                try:
                    srv.engine.remove_adapter(name)
                finally:
                    srv.engine.resume()

            await asyncio.to_thread(drop)
            await srv._fan_out("/v1/unload_lora_adapter", {"lora_name": name}, request)
            return {"status": "ok", "lora_name": name}

        @app.post("/detokenize")
        async def detokenize(request: Request):
            body = await request.json()
            return {"prompt": srv.tok.decode([int(t) for t in body.get("tokens", [])])}

        @app.post("/tokenize")
        async def tokenize(request: Request):
            body = await request.json()
            ids = srv._render_chat(body) if "messages" in body else srv.tok.encode(body.get("prompt", ""))
            return {"tokens": ids, "count": len(ids), "max_model_len": srv.engine.max_model_len}

        @app.post("/v1/chat/completions")
        async def chat(request: Request):
            srv._auth(request)
            body = await request.json()
            adapter = srv._route(body.get("model"))
            idx = srv._pick_replica() if srv.peers and not request.headers.get("x-art-routed") else 0
            if idx:
                return await srv._forward(idx, "/v1/chat/completions", body, request)
            try:
                prompt_ids = srv._render_chat(body)
            except Exception as e:
                raise HTTPException(status_code=400, detail=f"cannot render chat template: {e}") from e
            if body.get("truncate_prompt_tokens"):              # keep the end of an over-long prompt
                prompt_ids = prompt_ids[-int(body["truncate_prompt_tokens"]):]
            if len(prompt_ids) + 1 >= srv.engine.max_model_len:
                raise HTTPException(status_code=400, detail=f"prompt has {len(prompt_ids)} tokens; the maximum context "
                                                            f"length is {srv.engine.max_model_len}")
            params = srv._params(body, len(prompt_ids))
            want_prompt_lps = bool(body.get("prompt_logprobs")) and not body.get("stream")
            forced = srv._forced_tool_call(body)
            if forced is not None:
                params.guided_choice = [forced]       # the call is teacher-forced and comes back with its log-probs
            elif not params.guided_choice and srv._has_constraint(body):
                params.guided_regex = await asyncio.to_thread(srv._guided_regex, body)
                if params.guided_regex is not None:
                    await asyncio.to_thread(srv._ensure_masker)
            demanded = forced is not None or (params.guided_regex or "").startswith("<tool_call>")
            rid = "chatcmpl-" + uuid.uuid4().hex
            srv._log_request(rid, body, prompt_ids, params)
            model_name = body.get("model") or srv.base_model_name
            tools_on = bool(body.get("tools")) and body.get("tool_choice") != "none" and (srv.auto_tools or demanded)
            if body.get("stream"):
                include_usage = bool((body.get("stream_options") or {}).get("include_usage"))
                return StreamingResponse(srv._counted(srv._chat_stream(request, rid, model_name, prompt_ids, params, adapter,
                                                                       tools_on, include_usage)),
                                         media_type="text/event-stream")
            srv._load[0] += 1
            try:
                return JSONResponse(await srv._chat_full(request, rid, model_name, prompt_ids, params, adapter, tools_on,
                                                         want_prompt_lps))
            finally:
                srv._load[0] -= 1

        @app.post("/v1/completions")
        async def completions(request: Request):
            srv._auth(request)
            body = await request.json()
            adapter = srv._route(body.get("model"))
            idx = srv._pick_replica() if srv.peers and not request.headers.get("x-art-routed") else 0
            if idx:
                return await srv._forward(idx, "/v1/completions", body, request)
            prompts = srv._completion_prompts(body.get("prompt", ""))
            if body.get("truncate_prompt_tokens"):
                prompts = [p[-int(body["truncate_prompt_tokens"]):] for p in prompts]
            params = srv._params(body, max(len(p) for p in prompts))
            for p in prompts:
                if len(p) + 1 >= srv.engine.max_model_len:
                    raise HTTPException(status_code=400, detail=f"prompt has {len(p)} tokens; the maximum context length "
                                                                f"is {srv.engine.max_model_len}")
            if not params.guided_choice and srv._has_constraint({**body, "tool_choice": None}):
                params.guided_regex = await asyncio.to_thread(srv._guided_regex, {**body, "tool_choice": None})
                if params.guided_regex is not None:
                    await asyncio.to_thread(srv._ensure_masker)
            rid = "cmpl-" + uuid.uuid4().hex
            model_name = body.get("model") or srv.base_model_name
            srv._log_request(rid, body, prompts[0], params)
            echo = bool(body.get("echo"))
            if body.get("stream"):
                include_usage = bool((body.get("stream_options") or {}).get("include_usage"))
                return StreamingResponse(srv._counted(srv._completion_stream(rid, model_name, prompts, params, adapter, echo,
                                                                             include_usage)),
                                         media_type="text/event-stream")
            info: dict = {}
            srv._load[0] += 1
            try:
                outs = await asyncio.gather(*[srv._collect(request, p, params, adapter, info) for p in prompts])
                heads = await asyncio.gather(*[srv._echo_part(p, adapter, params) for p in prompts]) if echo else None
            finally:
                srv._load[0] -= 1
            choices = []
            for pi, out in enumerate(outs):
                for i, (ids, lps, reason, tops) in enumerate(out):
                    lpo = {"tokens": [srv._token_str(t) for t in ids], "token_logprobs": list(lps)}
                    if params.top_logprobs > 0:
                        lpo["top_logprobs"] = [{srv._token_str(t): l for t, l in (top or []) if t >= 0} for top in tops]
                    text = srv._cut_at_stop(srv.tok.decode(ids, skip_special_tokens=params.skip_special_tokens), params)
                    if echo:        # the prompt comes back in front, its tokens with their log-probs (None for the first)
                        h_text, h_tokens, h_lps = heads[pi]
                        text = h_text + text
                        lpo["tokens"] = h_tokens + lpo["tokens"]
                        lpo["token_logprobs"] = h_lps + lpo["token_logprobs"]
                        if "top_logprobs" in lpo:
                            lpo["top_logprobs"] = [None] * len(h_tokens) + lpo["top_logprobs"]
                    choices.append({"index": pi * params.n + i, "text": text, "finish_reason": reason, "logprobs": lpo})
            comp = sum(len(o[0]) for out in outs for o in out)
            return {"id": rid, "object": "text_completion", "created": _now(), "model": model_name, "choices": choices,
                    "usage": srv._usage(sum(len(p) for p in prompts), comp, info)}

        return app

    def _completion_prompts(self, prompt) -> list[list[int]]:
        """``prompt`` of ``/v1/completions``: a string, a list of token ids, or a list of either (one request each)."""
        def one(p) -> list[int]:
            if isinstance(p, str):
                return self.tok.encode(p)
            if isinstance(p, list) and all(isinstance(t, int) for t in p):
                return list(p)
            raise HTTPException(status_code=400, detail="prompt must be a string, a list of token ids, or a list of those")

        if isinstance(prompt, list) and prompt and not isinstance(prompt[0], int):
            out = [one(p) for p in prompt]
        else:
            out = [one(prompt)]
        if any(not p for p in out):
            raise HTTPException(status_code=400, detail="empty prompt")
        return out

    async def _echo_part(self, prompt_ids: list[int], adapter, params: SamplingParams) -> tuple[str, list[str], list]:
        """Text, token strings and log-probs (None for the first token) of a prompt that ``echo`` sends back."""
        lps: list = [None]
        if len(prompt_ids) > 1:
            lps += await self.engine.score(prompt_ids[:1], prompt_ids[1:], adapter)
        return self.tok.decode(prompt_ids, skip_special_tokens=True), [self._token_str(t) for t in prompt_ids], lps

    async def _completion_stream(self, rid, model_name, prompts, params, adapter, echo: bool, include_usage: bool
                                 ) -> AsyncIterator[str]:
        """Event stream of ``/v1/completions``: one chunk per scheduler step and choice with the new text, the tokens and
        their log-probs; choices of several prompts are numbered prompt-major."""
        def chunk(choices: list[dict], usage: dict | None = None) -> str:
            d = {"id": rid, "object": "text_completion", "created": _now(), "model": model_name, "choices": choices}
            if include_usage:
                d["usage"] = usage
            return "data: " + json.dumps(d) + "\n\n"

        q: asyncio.Queue = asyncio.Queue()
        info: dict = {}

        async def pump(pi: int, i: int):
            try:
                async for items in self._run_steps(prompts[pi], params, adapter, i, info):
                    for part in ([[it] for it in items] if self.stream_per_token else [items]):
                        await q.put((pi * params.n + i, part))
            except BaseException as e:  # noqa: BLE001
                await q.put(e)
            finally:
                await q.put((pi * params.n + i, None))

        tasks = [asyncio.create_task(pump(pi, i)) for pi in range(len(prompts)) for i in range(params.n)]
        live = len(tasks)
        bufs: dict[int, list[int]] = {k: [] for k in range(live)}
        decs = {k: IncrementalDecoder(self.tok, params.skip_special_tokens) for k in range(live)}
        sent: dict[int, int] = {k: 0 for k in range(live)}
        completion_tokens = 0
        try:
            if echo:
                for pi, p in enumerate(prompts):
                    text, tokens, lps = await self._echo_part(p, adapter, params)
                    for i in range(params.n):
                        yield chunk([{"index": pi * params.n + i, "text": text, "finish_reason": None,
                                      "logprobs": {"tokens": tokens, "token_logprobs": lps}}])
            while live:
                item = await q.get()
                if isinstance(item, BaseException):
                    raise item
                k, events = item
                if events is None:
                    live -= 1
                    continue
                lpo = None
                fin, why = False, None
                for _, tid, lp, fin, why, top in events:
                    if tid is not None:
                        completion_tokens += 1
                        bufs[k].append(tid)
                        if lpo is None:
                            lpo = {"tokens": [], "token_logprobs": []}
                            if params.top_logprobs > 0:
                                lpo["top_logprobs"] = []
                        lpo["tokens"].append(self._token_str(tid))
                        lpo["token_logprobs"].append(lp)
                        if params.top_logprobs > 0:
                            lpo["top_logprobs"].append({self._token_str(t): l for t, l in (top or []) if t >= 0})
                if lpo is not None:
                    decs[k].extend([t[1] for t in events if t[1] is not None and t[1] != self.engine.eos])
                full = self._cut_at_stop(decs[k].final() if fin else decs[k].text, params)
                upto = len(full) if fin else len(full) - self._held_back(full, params)
                text = ""
                if upto > sent[k]:
                    text, sent[k] = full[sent[k]:upto], upto
                yield chunk([{"index": k, "text": text, "finish_reason": (why or "stop") if fin else None, "logprobs": lpo}])
            if include_usage:
                yield chunk([], self._usage(sum(len(p) for p in prompts), completion_tokens, info))
            yield "data: [DONE]\n\n"
        finally:
            for t in tasks:
                t.cancel()

    async def _counted(self, agen):
        """Count a locally served stream as load of this replica while it runs."""
        self._load[0] += 1
        try:
            async for item in agen:
                yield item
        finally:
            self._load[0] -= 1

    # -- non-streaming ----------------------------------------------------------------------------------
    async def _collect(self, request: Request, prompt_ids, params: SamplingParams, adapter, info: dict | None = None):

        async def one(i: int):
            if not params.guided_choice and not params.stop and hasattr(self.engine, "complete"):
                # nothing has to look at the tokens on their way: let the engine run the request to its end
                seq_params = SamplingParams(**{**params.__dict__, "n": 1,
                                               "seed": None if params.seed is None else params.seed + i})
                seq = await self.engine.complete(prompt_ids, seq_params, adapter)
                if info is not None:
                    info["cached_tokens"] = max(info.get("cached_tokens", 0), getattr(seq, "prefix_hit_tokens", 0))
                return list(seq.output_ids), list(seq.logprobs), seq.finish_reason or "stop", list(seq.top_logprobs)
            ids, lps, tops, reason = [], [], [], "stop"
            async for _, tid, lp, fin, why, top in self._run_one(prompt_ids, params, adapter, i, info):
                if tid is not None:
                    ids.append(tid)
                    lps.append(lp)
                    tops.append(top)
                if fin:
                    reason = why or "stop"
            return ids, lps, reason, tops

        tasks = [asyncio.create_task(one(i)) for i in range(params.n)]
        watcher = asyncio.create_task(self._watch_disconnect(request, tasks))
        try:
            return await asyncio.gather(*tasks)
        except asyncio.CancelledError:
            raise HTTPException(status_code=499, detail="client disconnected") from None
        finally:
            watcher.cancel()

    async def _watch_disconnect(self, request: Request, tasks: list[asyncio.Task]) -> None:
        try:
            while True:
                if await request.is_disconnected():
                    for t in tasks:
                        t.cancel()
                    return
                await asyncio.sleep(0.25)
        except asyncio.CancelledError:
            pass
        except Exception:
            pass

    @staticmethod
    def _cut_at_stop(text: str, params: SamplingParams | None) -> str:
        """The text up to the first stop string (the string itself only with ``include_stop_str_in_output``): a request
        that ended on a stop string returns nothing past it, although the token that completed it may reach further."""
        if params is None or not params.stop:
            return text
        hits = [(text.find(s), s) for s in params.stop if s and s in text]
        if not hits:
            return text
        at, s_ = min(hits)
        return text[:at + (len(s_) if params.include_stop_str_in_output else 0)]

    @staticmethod
    def _held_back(text: str, params: SamplingParams | None) -> int:
        """Characters at the end of ``text`` that may be the beginning of a stop string and are therefore not streamed
        yet (they are sent, or cut, once the next tokens decide)."""
        if params is None or not params.stop:
            return 0
        keep = 0
        for s_ in params.stop:
            for n in range(min(len(s_) - 1, len(text)), 0, -1):
                if text.endswith(s_[:n]):
                    keep = max(keep, n)
                    break
        return keep

    def _strip_eos(self, ids: list[int]) -> list[int]:
        eos = self.engine.eos
        return ids[:-1] if ids and eos is not None and ids[-1] == eos else ids

    def _usage(self, n_prompt: int, n_completion: int, info: dict | None = None) -> dict:
        u: dict[str, Any] = {"prompt_tokens": n_prompt, "completion_tokens": n_completion,
                             "total_tokens": n_prompt + n_completion}
        if self.prompt_tokens_details:
            u["prompt_tokens_details"] = {"cached_tokens": int((info or {}).get("cached_tokens", 0))}
        return u

    def _log_request(self, rid: str, body: dict, prompt_ids: list[int], params: SamplingParams) -> None:
        if not self.log_requests:
            return
        n = self.max_log_len
        text = body.get("prompt") if isinstance(body.get("prompt"), str) else None
        if text is None and "messages" in body:
            text = " | ".join(str(m.get("content")) for m in body["messages"])
        ids = prompt_ids if n is None else prompt_ids[:n]
        _log.info("request %s: model=%s n=%d max_tokens=%d temperature=%s prompt=%r prompt_token_ids=%s", rid,
                  body.get("model"), params.n, params.max_tokens, params.temperature,
                  text if n is None or text is None else text[:n], ids)

    def _message_from(self, ids: list[int], tools_on: bool, reason: str, params: SamplingParams | None = None
                      ) -> tuple[dict, str]:
        skip = True if params is None else params.skip_special_tokens
        text = self._cut_at_stop(self.tok.decode(self._strip_eos(ids), skip_special_tokens=skip), params)
        msg: dict[str, Any] = {"role": self.role, "content": text}
        if self.reasoning is not None:
            r, text = split_reasoning(text, self.reasoning)
            msg["reasoning_content"] = r or None
            msg["content"] = text
            if text is None:
                return msg, reason
        if tools_on:
            content, calls = self.tool_parser.extract(text)
            if calls:
                msg["content"] = content
                msg["tool_calls"] = calls
                reason = "tool_calls"
        return msg, reason

    async def _chat_full(self, request, rid, model_name, prompt_ids, params, adapter, tools_on,
                         prompt_logprobs: bool = False) -> dict:
        info: dict = {}
        out = await self._collect(request, prompt_ids, params, adapter, info)
        choices = []
        for i, (ids, lps, reason, tops) in enumerate(out):
            msg, reason = self._message_from(ids, tools_on, reason, params)
            choices.append({"index": i, "message": msg, "finish_reason": reason,
                            "logprobs": {"content": [self._logprob_entry(t, lp, top) for t, lp, top in zip(ids, lps, tops)]}})
        comp = sum(len(o[0]) for o in out)
        resp = {"id": rid, "object": "chat.completion", "created": _now(), "model": model_name, "choices": choices,
                "usage": self._usage(len(prompt_ids), comp, info)}
        if prompt_logprobs:
            resp["prompt_logprobs"] = await self._prompt_logprobs(prompt_ids, adapter)
        return resp

    async def _prompt_logprobs(self, prompt_ids: list[int], adapter) -> list:
        """Log-probability of every prompt token given the ones before it (None for the first), in the shape the
        reference's engine returns for ``prompt_logprobs``: one ``{token_id: {"logprob", "decoded_token"}}`` per token."""
        _, _, lps = await self._echo_part(prompt_ids, adapter, None)
        return [None if lp is None else {str(t): {"logprob": lp, "decoded_token": self.tok.decode([t])}}
                for t, lp in zip(prompt_ids, lps)]

    # -- streaming --------------------------------------------------------------------------------------
    async def _chat_stream(self, request, rid, model_name, prompt_ids, params, adapter, tools_on, include_usage
                           ) -> AsyncIterator[str]:
        def chunk(choices: list[dict], usage: dict | None = None) -> str:
            d = {"id": rid, "object": "chat.completion.chunk", "created": _now(), "model": model_name, "choices": choices}
            if include_usage:
                d["usage"] = usage
            return "data: " + json.dumps(d) + "\n\n"

        q: asyncio.Queue = asyncio.Queue()
        info: dict = {}

        async def pump(i: int):
            try:
                async for items in self._run_steps(prompt_ids, params, adapter, i, info):
                    if self.stream_per_token:
                        for it in items:
                            await q.put([it])
                    else:
                        await q.put(items)     # the tokens of one scheduler step: one chunk of the stream
            except BaseException as e:  # noqa: BLE001
                await q.put(e)
            finally:
                await q.put((i, "done"))

        def visible(dec: IncrementalDecoder, done: bool) -> tuple[str, str]:
            """(reasoning, content) of a choice so far that may be sent: whole characters only, and without a possible
            beginning of a stop string or of a reasoning tag at the end, which wait for the next token."""
            full = self._cut_at_stop(dec.final() if done else dec.text, params)
            if self.reasoning is None:
                return "", full if done else full[:len(full) - self._held_back(full, params)]
            r, c = split_reasoning(full, self.reasoning, done)
            if c is None:
                return r, ""
            if not done:
                c = c[:len(c) - self._held_back(c, params)]
            return r, c

        tasks = [asyncio.create_task(pump(i)) for i in range(params.n)]
        live = params.n
        completion_tokens = 0
        bufs: dict[int, list[int]] = {i: [] for i in range(params.n)}
        decs = {i: IncrementalDecoder(self.tok, params.skip_special_tokens) for i in range(params.n)}
        sent_text: dict[int, int] = {i: 0 for i in range(params.n)}
        sent_reason: dict[int, int] = {i: 0 for i in range(params.n)}
        try:
            for i in range(params.n):
                yield chunk([{"index": i, "delta": {"role": self.role, "content": ""}, "logprobs": None, "finish_reason": None}])
            while live:
                item = await q.get()
                if isinstance(item, BaseException):
                    raise item
                if isinstance(item, tuple):
                    live -= 1
                    continue
                if not item:
                    continue
                i = item[0][0]
                delta: dict[str, Any] = {}
                entries = []
                fin, why = False, None
                for _, tid, lp, fin, why, top in item:
                    if tid is not None:
                        completion_tokens += 1
                        bufs[i].append(tid)
                        entries.append(self._logprob_entry(tid, lp, top))
                if entries:
                    decs[i].extend([t[1] for t in item if t[1] is not None and t[1] != self.engine.eos])
                lps = {"content": entries} if entries else None
                if not tools_on and (entries or fin):
                    r, c = visible(decs[i], bool(fin))
                    if len(r) > sent_reason[i]:
                        delta["reasoning_content"] = r[sent_reason[i]:]
                        sent_reason[i] = len(r)
                    if len(c) > sent_text[i]:
                        delta["content"] = c[sent_text[i]:]
                        sent_text[i] = len(c)
                reason = None
                if fin:
                    reason = why or "stop"
                    if tools_on:   # tool calls are parsed once the choice is complete; log-probs were streamed per token
                        msg, reason = self._message_from(bufs[i], True, reason, params)
                        if msg.get("reasoning_content"):
                            delta["reasoning_content"] = msg["reasoning_content"]
                        if msg.get("content"):
                            delta["content"] = msg["content"]
                        if msg.get("tool_calls"):
                            delta["tool_calls"] = [{"index": k, **c} for k, c in enumerate(msg["tool_calls"])]
                yield chunk([{"index": i, "delta": delta, "logprobs": lps, "finish_reason": reason}])
            if include_usage:
                yield chunk([], self._usage(len(prompt_ids), completion_tokens, info))
            yield "data: [DONE]\n\n"
        finally:
            for t in tasks:   # a disconnecting client lands here: abort only this request's sequences
                t.cancel()


def route_logs_to_file(path: str, level: int = logging.INFO) -> dict:
    """Sends the engine's and the server's log records to ``path`` (appending; one handler per path however often this
    is called) and returns a uvicorn ``log_config`` that sends uvicorn's own records there too, like the reference's
    engine log (src/art/local/vllm.py:335-382)."""
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    lg = logging.getLogger("art_b200.engine")
    path = os.path.abspath(path)
    if not any(isinstance(h, logging.FileHandler) and h.baseFilename == path for h in lg.handlers):
        h = logging.FileHandler(path)
        h.setFormatter(logging.Formatter("%(levelname)s %(asctime)s %(name)s] %(message)s", "%m-%d %H:%M:%S"))
        lg.addHandler(h)
    lg.setLevel(min(level, lg.level) if lg.level else level)
    from uvicorn.config import LOGGING_CONFIG

    handler = {"formatter": "default", "class": "logging.FileHandler", "filename": path}
    return {**LOGGING_CONFIG, "handlers": {"default": dict(handler), "access": {**handler, "formatter": "access"}}}


def serve_kwargs(sargs: dict) -> dict:
    """The listener's part of a ``ServerArgs`` dictionary as keyword arguments of :func:`serve`."""
    out = {k: sargs[k] for k in ("ssl_keyfile", "ssl_certfile", "ssl_ca_certs", "ssl_cert_reqs") if sargs.get(k) is not None}
    if sargs.get("uvicorn_log_level"):
        out["log_level"] = sargs["uvicorn_log_level"]
    return out


async def serve(server: OpenAIServer, host: str = "0.0.0.0", port: int = 8000, log_level: str = "warning",
                ready: asyncio.Event | None = None, **listener):
    """Run the app with uvicorn inside the current event loop until cancelled.  ``listener``: further keyword
    arguments of ``uvicorn.Config`` (TLS: ``ssl_keyfile``, ``ssl_certfile``, ``ssl_ca_certs``, ``ssl_cert_reqs``)."""
    import uvicorn

    config = uvicorn.Config(server.app, host=host, port=port, log_level=log_level, access_log=False,
                            root_path=server.root_path, **listener)
    uv = uvicorn.Server(config)
    uv.install_signal_handlers = lambda: None  # type: ignore[method-assign]
    task = asyncio.create_task(uv.serve())
    while not uv.started and not task.done():
        await asyncio.sleep(0.02)
    if ready is not None:
        ready.set()
    try:
        await task
    except asyncio.CancelledError:
        uv.should_exit = True
        await asyncio.sleep(0)
        raise
    return uv
