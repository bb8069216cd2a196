"""Teacher-forcing helpers (parity: reference ``src/art/guided_completion.py:12-71``).

Given a teacher's completion, build request parameters that force a student served by the
rollout engine to reproduce it: ``guided_choice`` for plain text, or a tool whose JSON
schema admits exactly the teacher's arguments plus a forced ``tool_choice``.
"""
from __future__ import annotations

import json
from copy import deepcopy
from typing import Iterable, Literal

from openai.types.chat.chat_completion import ChatCompletion
from pydantic import create_model


def freeze_tool_schema(tool: dict, fixed_args: dict) -> dict:
    """Clone ``tool`` with a parameter schema whose every field is a one-value enum."""
    fields = {name: (Literal[value], ...) for name, value in fixed_args.items()}  # type: ignore[valid-type]
    frozen = create_model(f"{tool['function']['name'].title()}FrozenArgs", **fields)
    out = deepcopy(tool)
    out["function"]["parameters"] = frozen.model_json_schema()
    return out


def get_guided_completion_params(completion: ChatCompletion, base_tools: Iterable[dict] | None = None):
    """Return ``(guided_choice, tool_choice, tool_params)`` for the first choice of ``completion``."""
    message = completion.choices[0].message
    if message.tool_calls:
        if base_tools is None:
            raise ValueError("No base tools provided")
        call = message.tool_calls[0]
        name = call.function.name
        try:
            tool = next(t for t in base_tools if t["function"]["name"] == name)
        except StopIteration:
            raise ValueError(f"tool {name!r} not among the base tools") from None
        tool_choice = {"type": "function", "function": {"name": name}}
        return None, tool_choice, [freeze_tool_schema(tool, json.loads(call.function.arguments))]
    return [message.content], None, None
