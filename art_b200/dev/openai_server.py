"""Completion-server configuration (parity: reference ``src/art/dev/openai_server.py:7-125``)."""
from __future__ import annotations

import json
from typing import Literal

from typing_extensions import TypedDict

from .engine import EngineArgs


class ServerArgs(TypedDict, total=False):
    host: str | None
    port: int
    uvicorn_log_level: Literal["debug", "info", "warning", "error", "critical", "trace"]
    allow_credentials: bool
    allowed_origins: str
    allowed_methods: str
    allowed_headers: str
    api_key: str | None
    lora_modules: list[str] | None  # 'name=path' or a JSON object {"name":..,"path":..}
    chat_template: str | None
    response_role: str | None
    root_path: str | None
    return_tokens_as_token_ids: bool
    enable_request_id_headers: bool
    enable_auto_tool_choice: bool
    tool_call_parser: str | None
    max_log_len: int | None
    disable_fastapi_docs: bool
    enable_prompt_tokens_details: bool
    enable_reasoning: bool
    reasoning_parser: str | None       # "deepseek_r1" (block open from the start), "qwen3", "granite"
    ssl_keyfile: str | None
    ssl_certfile: str | None
    ssl_ca_certs: str | None
    ssl_cert_reqs: int
    middleware: list[str]              # import paths of ASGI middleware classes or async (request, call_next) functions
    enable_server_load_tracking: bool  # GET /load
    # accepted for source compatibility, no effect here
    prompt_adapters: list[str] | None
    chat_template_content_format: Literal["auto", "string", "openai"]
    enable_ssl_refresh: bool
    disable_frontend_multiprocessing: bool
    tool_parser_plugin: str


class OpenAIServerConfig(TypedDict, total=False):
    """``log_file`` for the engine/server log, server arguments, and engine overrides."""

    log_file: str
    server_args: ServerArgs
    engine_args: EngineArgs


def parse_lora_module(spec: str) -> tuple[str, str]:
    """Accept both ``name=path`` and ``{"name":..,"path":..}`` forms."""
    spec = spec.strip()
    if spec.startswith("{"):
        d = json.loads(spec)
        return d["name"], d["path"]
    name, _, path = spec.partition("=")
    return name, path


def get_openai_server_config(model_name: str, base_model: str, log_file: str, lora_path: str,
                             config: OpenAIServerConfig | None = None) -> OpenAIServerConfig:
    config = config or OpenAIServerConfig()
    server_args = ServerArgs(
        api_key="default",
        lora_modules=[json.dumps({"name": model_name, "path": lora_path})],
        return_tokens_as_token_ids=True,
        enable_auto_tool_choice=True,
        tool_call_parser="hermes",
    )
    server_args.update(config.get("server_args", {}))
    engine_args = EngineArgs(model=base_model, served_model_name=base_model, num_scheduler_steps=16,
                             disable_log_requests=True, generation_config="vllm")
    engine_args.update(config.get("engine_args", {}))
    return OpenAIServerConfig(log_file=config.get("log_file", log_file), server_args=server_args,
                              engine_args=engine_args)
