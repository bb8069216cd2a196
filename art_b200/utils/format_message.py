"""Readable one-message rendering (parity: reference ``src/art/utils/format_message.py:4-19``)."""


def format_message(message: dict) -> str:
    role = str(message["role"]).capitalize()
    content = message.get("content", message.get("refusal", "")) or ""
    calls = "\n".join(f"{c['function']['name']}({c['function']['arguments']})" for c in (message.get("tool_calls") or []))
    sep = "\n" if content else ""
    return f"{role}:\n{content}{sep}{calls}"
