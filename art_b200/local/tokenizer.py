"""Tokenizer access.

``load_tokenizer(name)`` returns a Hugging Face tokenizer when ``name`` resolves locally
(a directory or a cached hub snapshot; the network is never required) and otherwise the
self-contained :class:`ByteChatTokenizer`, a byte-level tokenizer with a ChatML template.
The fallback is what random-init benchmark models and the CPU test-suite use; it
implements the subset of the HF interface the pipeline needs (``apply_chat_template``,
``encode``, ``decode``, ``vocab_size``, ``eos_token_id``).
"""
from __future__ import annotations

import json
import logging
from typing import Any

log = logging.getLogger(__name__)


class ByteChatTokenizer:
    """Byte-level tokenizer: ids 0..255 are bytes, then ``<|im_start|>``, ``<|im_end|>``, ``<|endoftext|>``.

    ``vocab_size`` may be larger than 259 so that the tokenizer can drive a model with a
    bigger embedding table; ids beyond the specials decode to ``<|extra_N|>`` strings.
    """

    IM_START, IM_END, EOT = 256, 257, 258

    def __init__(self, vocab_size: int = 512):
        if vocab_size < 259:
            raise ValueError("vocab_size must be at least 259")
        self.vocab_size = vocab_size
        self.eos_token_id = self.IM_END
        self.pad_token_id = self.EOT
        self.name_or_path = "byte-chat"
        self._specials = {self.IM_START: "<|im_start|>", self.IM_END: "<|im_end|>", self.EOT: "<|endoftext|>"}
        self._special_by_text = {v: k for k, v in self._specials.items()}

    def __len__(self) -> int:
        return self.vocab_size

    # -- text <-> ids -------------------------------------------------------------------
    def encode(self, text: str, add_special_tokens: bool = False) -> list[int]:
        ids: list[int] = []
        i = 0
        while i < len(text):
            if text[i] == "<" and text.startswith("<|", i):
                end = text.find("|>", i)
                if end != -1:
                    tok = text[i:end + 2]
                    if tok in self._special_by_text:
                        ids.append(self._special_by_text[tok])
                        i = end + 2
                        continue
                    if tok.startswith("<|extra_") and tok[8:-2].isdigit() and int(tok[8:-2]) < self.vocab_size:
                        ids.append(int(tok[8:-2]))
                        i = end + 2
                        continue
            ids.extend(text[i].encode("utf-8"))
            i += 1
        return ids

    def __call__(self, text: str, **_: Any) -> dict[str, list[int]]:
        ids = self.encode(text)
        return {"input_ids": ids, "attention_mask": [1] * len(ids)}

    def decode(self, ids, skip_special_tokens: bool = False) -> str:
        if isinstance(ids, int):
            ids = [ids]
        out: list[str] = []
        buf = bytearray()
        for t in ids:
            t = int(t)
            if t < 256:
                buf.append(t)
                continue
            if buf:
                out.append(buf.decode("utf-8", errors="replace"))
                buf = bytearray()
            if skip_special_tokens:
                continue
            out.append(self._specials.get(t, f"<|extra_{t}|>"))
        if buf:
            out.append(buf.decode("utf-8", errors="replace"))
        return "".join(out)

    def convert_ids_to_tokens(self, ids) -> list[str]:
        return [self.decode([i]) for i in ids]

    # -- chat template --------------------------------------------------------------------
    @staticmethod
    def _render_content(msg: dict) -> str:
        content = msg.get("content")
        if isinstance(content, list):
            content = "".join(p.get("text", "") for p in content if isinstance(p, dict))
        text = content or ""
        for call in msg.get("tool_calls") or []:
            fn = call["function"]
            args = fn["arguments"]
            if not isinstance(args, str):
                args = json.dumps(args)
            text += ("\n" if text else "") + "<tool_call>\n" + json.dumps({"name": fn["name"], "arguments": json.loads(args) if args else {}}) + "\n</tool_call>"
        return text

    def _segments(self, messages: list[dict], tools: list[dict] | None, add_generation_prompt: bool,
                  continue_final_message: bool = False):
        """Yield ``(text, is_assistant_content)`` pieces of the rendered conversation.  ``continue_final_message``
        leaves the last message open (no end marker), so that the model goes on writing it."""
        if tools:
            sys_txt = ("# Tools\n\nYou may call one or more functions to assist with the user query.\n\n"
                       "You are provided with function signatures within <tools></tools> XML tags:\n<tools>\n"
                       + "\n".join(json.dumps(t) for t in tools)
                       + "\n</tools>\n\nFor each function call, return a json object with function name and arguments "
                         "within <tool_call></tool_call> XML tags:\n<tool_call>\n"
                         '{"name": <function-name>, "arguments": <args-json-object>}\n</tool_call>')
            if messages and messages[0]["role"] == "system":
                first = dict(messages[0])
                first["content"] = self._render_content(first) + "\n\n" + sys_txt
                messages = [first] + list(messages[1:])
            else:
                messages = [{"role": "system", "content": sys_txt}] + list(messages)
        for idx, m in enumerate(messages):
            role = m["role"]
            if continue_final_message and idx == len(messages) - 1:
                yield f"<|im_start|>{role}\n", False
                yield self._render_content(m), role == "assistant"
                return
            if role == "tool":
                yield f"<|im_start|>user\n<tool_response>\n{self._render_content(m)}\n</tool_response><|im_end|>\n", False
                continue
            yield f"<|im_start|>{role}\n", False
            if role == "assistant":
                yield self._render_content(m) + "<|im_end|>", True
                yield "\n", False
            else:
                yield self._render_content(m) + "<|im_end|>\n", False
        if add_generation_prompt:
            yield "<|im_start|>assistant\n", False

    def apply_chat_template(self, messages: list[dict], tools: list[dict] | None = None, tokenize: bool = True,
                            add_generation_prompt: bool = False, return_dict: bool = False,
                            return_assistant_tokens_mask: bool = False, chat_template: str | None = None,
                            continue_final_message: bool = False, **kw: Any):
        """``chat_template``: a Jinja template used instead of the built-in ChatML layout (variables ``messages``,
        ``tools``, ``add_generation_prompt``, the special-token strings and any further keyword); a custom template has
        no assistant mask."""
        if chat_template:
            import jinja2.sandbox

            env = jinja2.sandbox.ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True)
            text = env.from_string(chat_template).render(
                messages=messages, tools=tools, add_generation_prompt=add_generation_prompt,
                bos_token="", eos_token=self._specials[self.IM_END], **kw)
            pieces = [(text, False)]
        else:
            if continue_final_message and add_generation_prompt:
                raise ValueError("continue_final_message and add_generation_prompt exclude each other")
            pieces = list(self._segments(list(messages), tools, add_generation_prompt, continue_final_message))
        if not tokenize:
            return "".join(p for p, _a in pieces)
        ids: list[int] = []
        amask: list[int] = []
        for text, is_asst in pieces:
            enc = self.encode(text)
            ids.extend(enc)
            amask.extend([1 if is_asst else 0] * len(enc))
        if not return_dict:
            return ids
        out = {"input_ids": ids, "attention_mask": [1] * len(ids)}
        if return_assistant_tokens_mask:
            out["assistant_masks"] = amask
        return out


_cache: dict[str, Any] = {}


def load_tokenizer(name: str, vocab_size: int | None = None):
    """HF tokenizer if available locally, else :class:`ByteChatTokenizer`."""
    key = f"{name}:{vocab_size}"
    if key in _cache:
        return _cache[key]
    tok = None
    if not name.startswith("random:") and not name.startswith("byte-chat"):
        try:
            from transformers import AutoTokenizer

            tok = AutoTokenizer.from_pretrained(name, local_files_only=True)
        except Exception as e:  # no local snapshot
            log.warning("tokenizer %r not available locally (%s); using the byte-level chat tokenizer", name, type(e).__name__)
    if tok is None:
        tok = ByteChatTokenizer(vocab_size or 512)
    _cache[key] = tok
    return tok
