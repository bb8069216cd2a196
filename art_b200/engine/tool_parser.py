"""Hermes-format tool-call parsing (``<tool_call>{"name": ..., "arguments": {...}}</tool_call>``),
the format the reference enables by default (``tool_call_parser="hermes"``,
``src/art/dev/openai_server.py:17-23``)."""
from __future__ import annotations

import json
import re
import uuid

_CALL = re.compile(r"<tool_call>\s*(.*?)\s*(?:</tool_call>|$)", re.DOTALL)


class HermesToolParser:
    def extract(self, text: str) -> tuple[str | None, list[dict]]:
        """Return ``(content, tool_calls)``; ``tool_calls`` is empty when none parse."""
        if "<tool_call>" not in text:
            return text, []
        calls = []
        for m in _CALL.finditer(text):
            try:
                obj = json.loads(m.group(1))
                name = obj["name"]
                args = obj.get("arguments", obj.get("parameters", {}))
            except (json.JSONDecodeError, KeyError, TypeError):
                continue
            calls.append({"id": "chatcmpl-tool-" + uuid.uuid4().hex[:24], "type": "function",
                          "function": {"name": name, "arguments": args if isinstance(args, str) else json.dumps(args)}})
        if not calls:
            return text, []
        content = text[: text.index("<tool_call>")]       # as written, like the reference's parser (no stripping)
        return (content or None), calls
