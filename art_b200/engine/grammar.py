"""Structured outputs: constrain a completion to a regular expression or a JSON schema.

The reference serves ``guided_json`` / ``guided_regex`` / ``response_format`` and named ``tool_choice`` through its
inference library (the request schema is inherited whole, src/art/local/vllm.py:234-247; the distillation helper
relies on it, src/art/guided_completion.py:12-26).  Here the pieces are:

* :func:`compile_regex`: a regular expression -> a deterministic automaton over UTF-8 *bytes* (tokens of byte-level
  vocabularies are byte strings, not character strings, and may end in the middle of a character);
* :func:`schema_to_regex`: a JSON schema -> such an expression (objects with their properties in declared order,
  optional properties, arrays with bounds, enums, constants, ``anyOf``, local ``$ref``, strings with length bounds or
  patterns; values without a schema are any JSON of bounded nesting depth);
* :class:`TokenMasker`: which tokens of a vocabulary may follow in a given automaton state.  The vocabulary is a byte
  trie that is walked together with the automaton, so a dead prefix prunes every token below it; the walk is native
  code (``csrc/engine/token_mask.cpp``) with a Python twin, and masks are cached per state;
* :class:`GrammarState`: the per-request cursor the scheduler advances token by token.

Sequences with a grammar are scheduled one decode step at a time (the next mask depends on the token just drawn),
like sequences with penalties.
"""
from __future__ import annotations

import ctypes
import json
from dataclasses import dataclass

import numpy as np

MAX_DFA_STATES = 50_000


# ------------------------------------------------------------------------------------------- regex -> AST
# AST nodes: ("set", mask) one byte out of a 256-bit mask; ("cat", [nodes]); ("alt", [nodes]); ("star", node);
# ("opt", node); ("eps",)

def _mask_of(byte_values) -> int:
    m = 0
    for b in byte_values:
        m |= 1 << b
    return m


def _lit(data: bytes):
    return ("cat", [("set", 1 << b) for b in data]) if len(data) != 1 else ("set", 1 << data[0])


_CONT = _mask_of(range(0x80, 0xC0))
# any character that is not ASCII, as UTF-8 (over-long forms and surrogates are not excluded: the text comes out of a
# tokenizer's vocabulary, not from an adversary)
_NON_ASCII = ("alt", [
    ("cat", [("set", _mask_of(range(0xC2, 0xE0))), ("set", _CONT)]),
    ("cat", [("set", _mask_of(range(0xE0, 0xF0))), ("set", _CONT), ("set", _CONT)]),
    ("cat", [("set", _mask_of(range(0xF0, 0xF5))), ("set", _CONT), ("set", _CONT), ("set", _CONT)]),
])
_CLASS_ESC = {"d": _mask_of(range(48, 58)), "s": _mask_of(b" \t\n\r\f\v"),
              "w": _mask_of(list(range(48, 58)) + list(range(65, 91)) + list(range(97, 123)) + [95])}
_CHAR_ESC = {"n": "\n", "t": "\t", "r": "\r", "f": "\f", "v": "\v", "0": "\0"}
_ASCII = (1 << 128) - 1


class RegexError(ValueError):
    pass


class _Parser:
    """Recursive descent over the usual syntax: literals, ``.``, escapes (``\\d \\w \\s`` and their negations, ``\\n`` ...,
    ``\\xHH``, ``\\uHHHH``), classes with ranges and negation, groups (capturing or ``(?:``), ``|``, and the quantifiers
    ``* + ? {m} {m,} {m,n}`` (lazy marks are accepted and ignored: only the language matters).  Anchors ``^`` / ``$``
    at the ends are dropped: the whole completion always has to match."""

    def __init__(self, src: str):
        self.s, self.i = src, 0

    def parse(self):
        node = self.alt()
        if self.i != len(self.s):
            raise RegexError(f"unexpected {self.s[self.i]!r} at {self.i}")
        return node

    def peek(self) -> str | None:
        return self.s[self.i] if self.i < len(self.s) else None

    def alt(self):
        parts = [self.cat()]
        while self.peek() == "|":
            self.i += 1
            parts.append(self.cat())
        return parts[0] if len(parts) == 1 else ("alt", parts)

    def cat(self):
        items = []
        while self.peek() is not None and self.peek() not in "|)":
            items.append(self.repeat())
        if not items:
            return ("eps",)
        return items[0] if len(items) == 1 else ("cat", items)

    def repeat(self):
        node = self.atom()
        while True:
            c = self.peek()
            if c == "*":
                self.i += 1
                node = ("star", node)
            elif c == "+":
                self.i += 1
                node = ("cat", [node, ("star", node)])
            elif c == "?":
                self.i += 1
                node = ("opt", node)
            elif c == "{":
                j = self.s.find("}", self.i)
                body = self.s[self.i + 1:j] if j != -1 else ""
                lo_s, comma, hi_s = body.partition(",")
                if j == -1 or not lo_s.strip().isdigit() or (hi_s.strip() and not hi_s.strip().isdigit()):
                    raise RegexError(f"bad quantifier at {self.i}")
                self.i = j + 1
                lo = int(lo_s)
                hi = lo if not comma else (int(hi_s) if hi_s.strip() else None)
                if hi is not None and hi < lo:
                    raise RegexError("quantifier with max < min")
                if (hi if hi is not None else lo) > 1000:
                    raise RegexError("quantifier bound above 1000")
                seq = [node] * lo
                if hi is None:
                    seq.append(("star", node))
                else:
                    tail = ("eps",)
                    for _ in range(hi - lo):         # (x(x(x)?)?)? keeps the automaton linear in hi
                        tail = ("opt", ("cat", [node, tail]) if tail != ("eps",) else node)
                    if hi > lo:
                        seq.append(tail)
                node = ("cat", seq) if seq else ("eps",)
            else:
                return node
            if self.peek() == "?" and c in "*+?{":      # lazy mark
                self.i += 1

    def atom(self):
        c = self.peek()
        self.i += 1
        if c == "(":
            if self.s.startswith("?:", self.i):
                self.i += 2
            elif self.s.startswith("?", self.i):
                raise RegexError("look-around and named groups are not supported")
            node = self.alt()
            if self.peek() != ")":
                raise RegexError("missing )")
            self.i += 1
            return node
        if c == "[":
            return self.char_class()
        if c == ".":
            return ("alt", [("set", _ASCII & ~(1 << 10)), _NON_ASCII])
        if c == "^" and self.i == 1:
            return ("eps",)
        if c == "$" and self.i == len(self.s):
            return ("eps",)
        if c == "\\":
            kind, val = self.escape()
            if kind == "mask":
                return ("set", val)
            if kind == "negmask":
                return ("alt", [("set", _ASCII & ~val), _NON_ASCII])
            return _lit(val.encode("utf-8"))
        if c in "*+?{":
            raise RegexError(f"nothing to repeat at {self.i - 1}")
        return _lit(c.encode("utf-8"))

    def escape(self):
        c = self.peek()
        if c is None:
            raise RegexError("dangling backslash")
        self.i += 1
        if c in _CLASS_ESC:
            return "mask", _CLASS_ESC[c]
        if c.lower() in _CLASS_ESC and c.isupper():
            return "negmask", _CLASS_ESC[c.lower()]
        if c in _CHAR_ESC:
            return "char", _CHAR_ESC[c]
        if c in "bBAZzGpPkK" or (c.isdigit() and c != "0"):
            raise RegexError(f"\\{c} (boundaries, back-references, Unicode properties) is not supported")
        if c in "xu":
            n = 2 if c == "x" else 4
            hexs = self.s[self.i:self.i + n]
            if len(hexs) != n or any(h not in "0123456789abcdefABCDEF" for h in hexs):
                raise RegexError("bad hexadecimal escape")
            self.i += n
            return "char", chr(int(hexs, 16))
        return "char", c

    def char_class(self):
        neg = self.peek() == "^"
        if neg:
            self.i += 1
        mask, wide, first = 0, [], True
        while True:
            c = self.peek()
            if c is None:
                raise RegexError("missing ]")
            if c == "]" and not first:
                self.i += 1
                break
            first = False
            self.i += 1
            if c == "\\":
                kind, val = self.escape()
                if kind == "mask":
                    mask |= val
                    continue
                if kind == "negmask":
                    mask |= _ASCII & ~val
                    wide.append(None)
                    continue
                c = val
            if self.peek() == "-" and self.i + 1 < len(self.s) and self.s[self.i + 1] != "]":
                self.i += 1
                hi = self.peek()
                self.i += 1
                if hi == "\\":
                    kind, hi = self.escape()
                    if kind != "char":
                        raise RegexError("bad range")
                lo_o, hi_o = ord(c), ord(hi)
                if hi_o < lo_o:
                    raise RegexError("bad range")
                for o in range(lo_o, min(hi_o, 127) + 1):
                    mask |= 1 << o
                if hi_o > 127:
                    if hi_o - max(lo_o, 128) > 4096:
                        raise RegexError("non-ASCII range too wide")
                    wide.extend(chr(o) for o in range(max(lo_o, 128), hi_o + 1))
            elif ord(c) < 128:
                mask |= 1 << ord(c)
            else:
                wide.append(c)
        if neg:
            if any(w is not None for w in wide):
                raise RegexError("negated classes may exclude ASCII characters only")
            return ("alt", [("set", _ASCII & ~mask), _NON_ASCII])
        alts = [("set", mask)] if mask else []
        if None in wide:
            alts.append(_NON_ASCII)
        alts.extend(_lit(w.encode("utf-8")) for w in wide if w is not None)
        if not alts:
            raise RegexError("empty class")
        return alts[0] if len(alts) == 1 else ("alt", alts)


# ------------------------------------------------------------------------------------------- AST -> NFA -> DFA
@dataclass
class ByteDFA:
    """``trans[s, b]`` is the next state or -1; state 0 is the start."""
    trans: np.ndarray          # int32 [n_states, 256]
    accepting: np.ndarray      # bool [n_states]

    @property
    def n_states(self) -> int:
        return int(self.trans.shape[0])

    def walk(self, state: int, data: bytes) -> int:
        for b in data:
            if state < 0:
                return -1
            state = int(self.trans[state, b])
        return state

    def matches(self, text: str | bytes) -> bool:
        s = self.walk(0, text.encode("utf-8") if isinstance(text, str) else text)
        return s >= 0 and bool(self.accepting[s])


def _build_nfa(ast):
    eps: list[list[int]] = []
    edges: list[list[tuple[int, int]]] = []     # state -> [(mask, target)]

    def new() -> int:
        eps.append([])
        edges.append([])
        return len(eps) - 1

    def build(node) -> tuple[int, int]:
        kind = node[0]
        if kind == "eps":
            a = new()
            return a, a
        if kind == "set":
            a, b = new(), new()
            edges[a].append((node[1], b))
            return a, b
        if kind == "cat":
            first, last = build(node[1][0])
            for sub in node[1][1:]:
                a, b = build(sub)
                eps[last].append(a)
                last = b
            return first, last
        if kind == "alt":
            a, b = new(), new()
            for sub in node[1]:
                x, y = build(sub)
                eps[a].append(x)
                eps[y].append(b)
            return a, b
        if kind == "opt":
            a, b = new(), new()
            x, y = build(node[1])
            eps[a] += [x, b]
            eps[y].append(b)
            return a, b
        if kind == "star":
            a, b = new(), new()
            x, y = build(node[1])
            eps[a] += [x, b]
            eps[y] += [x, b]
            return a, b
        raise AssertionError(kind)

    import sys

    old = sys.getrecursionlimit()
    sys.setrecursionlimit(max(old, 20000))
    try:
        start, end = build(ast)
    finally:
        sys.setrecursionlimit(old)
    return start, end, eps, edges


def compile_regex(pattern: str) -> ByteDFA:
    """The automaton of ``pattern`` (the whole text must match)."""
    start, end, eps, edges = _build_nfa(_Parser(pattern).parse())

    def closure(states) -> frozenset:
        seen, stack = set(states), list(states)
        while stack:
            for t in eps[stack.pop()]:
                if t not in seen:
                    seen.add(t)
                    stack.append(t)
        return frozenset(seen)

    s0 = closure([start])
    index = {s0: 0}
    order = [s0]
    rows: list[list[int]] = []
    k = 0
    while k < len(order):
        cur = order[k]
        k += 1
        row = [-1] * 256
        out = [(m, t) for s in cur for (m, t) in edges[s]]
        if out:
            union = 0
            for m, _ in out:
                union |= m
            b = 0
            while union:
                if union & 1:
                    tgt = closure([t for (m, t) in out if (m >> b) & 1])
                    j = index.get(tgt)
                    if j is None:
                        if len(order) >= MAX_DFA_STATES:
                            raise RegexError(f"the expression needs more than {MAX_DFA_STATES} automaton states")
                        j = index[tgt] = len(order)
                        order.append(tgt)
                    row[b] = j
                union >>= 1
                b += 1
        rows.append(row)
    return ByteDFA(np.asarray(rows, dtype=np.int32).reshape(len(rows), 256),
                   np.asarray([end in s for s in order], dtype=bool))


# ------------------------------------------------------------------------------------------- JSON schema -> regex
WS = "[ ]?"
_STR_CHAR = r'([^"\\\x00-\x1f]|\\["\\/bfnrt]|\\u[0-9a-fA-F]{4})'
STRING = f'"{_STR_CHAR}*"'
INTEGER = r"-?(0|[1-9][0-9]*)"
NUMBER = INTEGER + r"(\.[0-9]+)?([eE][+-]?[0-9]+)?"
BOOLEAN = "(true|false)"
NULL = "null"
_FORMATS = {
    "date": r'"[0-9]{4}-(0[1-9]|1[0-2])-(0[1-9]|[12][0-9]|3[01])"',
    "time": r'"([01][0-9]|2[0-3]):[0-5][0-9]:[0-5][0-9](\.[0-9]+)?(Z|[+-][0-9]{2}:[0-9]{2})?"',
    "date-time": r'"[0-9]{4}-(0[1-9]|1[0-2])-(0[1-9]|[12][0-9]|3[01])T([01][0-9]|2[0-3]):[0-5][0-9]:[0-5][0-9](\.[0-9]+)?'
                 r'(Z|[+-][0-9]{2}:[0-9]{2})?"',
    "uuid": r'"[0-9a-fA-F]{8}-[0-9a-fA-F]{4}-[0-9a-fA-F]{4}-[0-9a-fA-F]{4}-[0-9a-fA-F]{12}"',
}


def int_range_regex(lo: int, hi: int) -> str:
    """The decimal integers ``lo..hi`` (no leading zeros, no ``-0``) as a regular expression."""
    if lo > hi:
        raise ValueError(f"empty integer range {lo}..{hi}")

    def group(alts: list[str]) -> str:
        return alts[0] if len(alts) == 1 else "(" + "|".join(alts) + ")"

    def same_len(a: str, b: str) -> list[str]:
        """Digit strings of one length between ``a`` and ``b`` (inner digits: zeros allowed)."""
        if a == b:
            return [a]
        if len(a) == 1:
            return [f"[{a}-{b}]"]
        n = len(a) - 1
        if a[0] == b[0]:
            return [a[0] + group(same_len(a[1:], b[1:]))]
        out = [a[0] + group(same_len(a[1:], "9" * n))]
        if int(b[0]) - int(a[0]) > 1:
            out.append(f"[{int(a[0]) + 1}-{int(b[0]) - 1}][0-9]{{{n}}}")
        out.append(b[0] + group(same_len("0" * n, b[1:])))
        return out

    def non_negative(a: int, b: int) -> list[str]:
        out: list[str] = []
        for nd in range(len(str(a)), len(str(b)) + 1):
            first = max(a, 10 ** (nd - 1) if nd > 1 else 0)
            last = min(b, 10 ** nd - 1)
            if first <= last:
                out += same_len(str(first), str(last))
        return out

    alts: list[str] = []
    if lo < 0:
        alts.append("-" + group(non_negative(max(1, -hi) if hi < 0 else 1, -lo)))
    if hi >= 0:
        alts += non_negative(max(lo, 0), hi)
    return group(alts)


def escape_literal(text: str) -> str:
    return "".join("\\" + c if c in r"\.[]{}()*+?|^$-" else c for c in text)


def any_json(depth: int = 3) -> str:
    """Any JSON value nested at most ``depth`` containers deep."""
    scalar = f"({STRING}|{NUMBER}|{BOOLEAN}|{NULL})"
    value = scalar
    for _ in range(depth):
        arr = rf"\[{WS}({value}({WS},{WS}{value})*)?{WS}\]"
        member = f"{STRING}{WS}:{WS}{value}"
        obj = rf"\{{{WS}({member}({WS},{WS}{member})*)?{WS}\}}"
        value = f"({scalar}|{arr}|{obj})"
    return value


def schema_to_regex(schema: dict | bool | str, *, any_depth: int = 2, max_ref_depth: int = 4) -> str:
    """A regular expression for the JSON texts that satisfy ``schema`` (a dictionary, its JSON text, or ``True``)."""
    if isinstance(schema, str):
        schema = json.loads(schema)
    root = schema if isinstance(schema, dict) else {}

    def resolve(ref: str) -> dict:
        if not ref.startswith("#/"):
            raise ValueError(f"only local references are supported, not {ref!r}")
        node = root
        for part in ref[2:].split("/"):
            node = node[part.replace("~1", "/").replace("~0", "~")]
        return node

    def conv(s, refs: int) -> str:
        if s is True or s == {} or s is None:
            return any_json(any_depth)
        if s is False:
            raise ValueError("a schema that admits nothing")
        if "$ref" in s:
            if refs >= max_ref_depth:
                raise ValueError(f"references nested deeper than {max_ref_depth} (recursive schemas are not regular)")
            return conv(resolve(s["$ref"]), refs + 1)
        if "const" in s:
            return escape_literal(json.dumps(s["const"], ensure_ascii=False))
        if "enum" in s:
            return "(" + "|".join(escape_literal(json.dumps(v, ensure_ascii=False)) for v in s["enum"]) + ")"
        for key in ("anyOf", "oneOf"):
            if key in s:
                return "(" + "|".join(conv(sub, refs) for sub in s[key]) + ")"
        if "allOf" in s:
            if len(s["allOf"]) == 1:
                return conv(s["allOf"][0], refs)
            raise ValueError("allOf with several members is not supported")
        t = s.get("type")
        if isinstance(t, list):
            return "(" + "|".join(conv({**s, "type": one}, refs) for one in t) + ")"
        if t is None:
            t = "object" if "properties" in s else ("array" if "items" in s else None)
            if t is None:
                return any_json(any_depth)
        if t == "string":
            if "pattern" in s:
                p = s["pattern"]
                p = p[1:] if p.startswith("^") else p
                p = p[:-1] if p.endswith("$") and not p.endswith("\\$") else p
                return f'"({p})"'
            if s.get("format") in _FORMATS:
                return _FORMATS[s["format"]]
            lo, hi = s.get("minLength"), s.get("maxLength")
            if lo is not None or hi is not None:
                return f'"{_STR_CHAR}{{{int(lo or 0)},{"" if hi is None else int(hi)}}}"'
            return STRING
        if t == "integer":
            lo, hi = s.get("minimum", s.get("exclusiveMinimum")), s.get("maximum", s.get("exclusiveMaximum"))
            if lo is not None and hi is not None:
                lo_i = int(lo) + (1 if "exclusiveMinimum" in s and "minimum" not in s else 0)
                hi_i = int(hi) - (1 if "exclusiveMaximum" in s and "maximum" not in s else 0)
                return int_range_regex(lo_i, hi_i)
            if lo is not None and lo >= 0:
                return "(0|[1-9][0-9]*)"
            return INTEGER
        if t == "number":
            return NUMBER
        if t == "boolean":
            return BOOLEAN
        if t == "null":
            return NULL
        if t == "array":
            item = conv(s.get("items", True), refs)
            lo, hi = int(s.get("minItems", 0)), s.get("maxItems")
            if hi is not None and int(hi) == 0:
                return rf"\[{WS}\]"
            more = f"({WS},{WS}{item})"
            rest = f"{more}{{{max(lo - 1, 0)},{'' if hi is None else int(hi) - 1}}}"
            body = f"{item}{rest}"
            return rf"\[{WS}{body}{WS}\]" if lo > 0 else rf"\[{WS}({body})?{WS}\]"
        if t == "object":
            props = s.get("properties") or {}
            if not props:
                extra = s.get("additionalProperties", True)
                if extra is False:
                    return rf"\{{{WS}\}}"
                value = conv(extra if isinstance(extra, dict) else True, refs)
                member = f"{STRING}{WS}:{WS}{value}"
                return rf"\{{{WS}({member}({WS},{WS}{member})*)?{WS}\}}"
            required = set(s.get("required") or [])
            names = list(props)
            members = [f'"{escape_literal(json.dumps(n, ensure_ascii=False)[1:-1])}"{WS}:{WS}{conv(props[n], refs)}'
                       for n in names]
            is_req = [n in required for n in names]
            first_req = next((i for i, r in enumerate(is_req) if r), len(names))
            alts = []
            for i in range(min(first_req, len(names) - 1) + 1):      # property i is the first one present
                pat = members[i]
                for j in range(i + 1, len(names)):
                    nxt = f"{WS},{WS}{members[j]}"
                    pat += nxt if is_req[j] else f"({nxt})?"
                alts.append(pat)
            body = "(" + "|".join(alts) + ")"
            if not required:
                body += "?"
            return rf"\{{{WS}{body}{WS}\}}"
        raise ValueError(f"unsupported schema type {t!r}")

    return conv(schema, 0)


# ------------------------------------------------------------------------------------------- vocabulary
def _gpt2_byte_decoder() -> dict[str, int]:
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return {chr(c): b for b, c in zip(bs, cs)}


def vocabulary_bytes(tokenizer) -> list[bytes]:
    """The byte string of every token id (``b""`` for special tokens and ids without text: they are never allowed
    inside a constrained completion).  Handles the in-tree byte tokenizer, byte-level BPE vocabularies (GPT-2 style
    byte-to-character table: Qwen, Llama 3) and SentencePiece-style vocabularies (``▁`` for a space, ``<0xNN>`` bytes)."""
    n = len(tokenizer)
    if getattr(tokenizer, "name_or_path", "") == "byte-chat" and hasattr(tokenizer, "IM_START"):
        return [bytes([i]) if i < 256 else b"" for i in range(n)]
    special = set(getattr(tokenizer, "all_special_ids", []) or [])
    added = getattr(tokenizer, "get_added_vocab", lambda: {})()
    special |= set(added.values())
    toks = tokenizer.convert_ids_to_tokens(list(range(n)))
    byte_level = any(t is not None and t.startswith("Ġ") for t in toks[:50000])
    dec = _gpt2_byte_decoder() if byte_level else None
    out: list[bytes] = []
    for i, t in enumerate(toks):
        if t is None or i in special:
            out.append(b"")
        elif dec is not None:
            try:
                out.append(bytes(dec[c] for c in t))
            except KeyError:
                out.append(b"")
        elif len(t) == 6 and t.startswith("<0x") and t.endswith(">"):
            out.append(bytes([int(t[3:5], 16)]))
        else:
            out.append(t.replace("▁", " ").encode("utf-8"))
    return out


class TokenMasker:
    """Allowed-token masks of one vocabulary under byte automata.  ``mask(dfa, state)`` is a bool array over token
    ids: token ``t`` is allowed when walking its bytes from ``state`` never leaves the automaton."""

    def __init__(self, vocab: list[bytes], eos_token_id: int | None = None, use_native: bool = True):
        self.vocab = vocab
        self.eos = eos_token_id
        self.n = len(vocab)
        self._native = None
        self._trie = None
        if use_native:
            try:
                self._native = _NativeTrie(vocab)
            except (OSError, AttributeError):
                self._native = None
        self._cache: dict[tuple[int, int], np.ndarray] = {}       # (automaton, state) -> bit-packed mask
        self._dfa_refs: dict[int, ByteDFA] = {}

    # -- Python twin of the native walk ----------------------------------------------------
    def _py_trie(self):
        if self._trie is None:
            children: list[dict[int, int]] = [{}]
            terminal: list[list[int]] = [[]]
            for tid, data in enumerate(self.vocab):
                if not data:
                    continue
                node = 0
                for b in data:
                    nxt = children[node].get(b)
                    if nxt is None:
                        nxt = len(children)
                        children[node][b] = nxt
                        children.append({})
                        terminal.append([])
                    node = nxt
                terminal[node].append(tid)
            self._trie = (children, terminal)
        return self._trie

    def _py_mask(self, dfa: ByteDFA, state: int) -> np.ndarray:
        children, terminal = self._py_trie()
        out = np.zeros(self.n, dtype=bool)
        trans = dfa.trans
        stack = [(0, state)]
        while stack:
            node, s = stack.pop()
            row = trans[s]
            for b, child in children[node].items():
                t = int(row[b])
                if t >= 0:
                    for tid in terminal[child]:
                        out[tid] = True
                    if children[child]:
                        stack.append((child, t))
        return out

    def mask(self, dfa: ByteDFA, state: int) -> np.ndarray:
        key = (id(dfa), state)
        packed = self._cache.get(key)
        if packed is not None:
            return np.unpackbits(packed, count=self.n).view(bool)
        self._dfa_refs[id(dfa)] = dfa          # keeps the id stable while its masks are cached
        m = self._native.mask(dfa, state) if self._native is not None else self._py_mask(dfa, state)
        if self.eos is not None and 0 <= self.eos < self.n:
            m[self.eos] = bool(dfa.accepting[state])
        if len(self._cache) > 4096:
            self._cache.clear()
            self._dfa_refs = {id(dfa): dfa}      # automata are pinned only while masks of theirs are cached
        self._cache[key] = np.packbits(m)        # one bit per token: 19 KB per state for a 150 k vocabulary
        return m


class _NativeTrie:
    def __init__(self, vocab: list[bytes]):
        from ..ops import _lib

        lib = _lib.runtime()
        vp, ci = ctypes.c_void_p, ctypes.c_int
        lib.artb_tm_create.argtypes = [vp, vp, ci]
        lib.artb_tm_create.restype = vp
        lib.artb_tm_destroy.argtypes = [vp]
        lib.artb_tm_mask.argtypes = [vp, vp, ci, ci, vp]
        lib.artb_tm_mask.restype = ci
        self._lib = lib
        offsets = np.zeros(len(vocab) + 1, dtype=np.int64)
        np.cumsum([len(v) for v in vocab], out=offsets[1:])
        blob = np.frombuffer(b"".join(vocab) or b"\0", dtype=np.uint8)
        self.n = len(vocab)
        self._h = lib.artb_tm_create(blob.ctypes.data, offsets.ctypes.data, self.n)
        if not self._h:
            raise OSError("token trie could not be built")

    def mask(self, dfa: ByteDFA, state: int) -> np.ndarray:
        out = np.zeros(self.n, dtype=np.uint8)
        trans = np.ascontiguousarray(dfa.trans, dtype=np.int32)
        rc = self._lib.artb_tm_mask(self._h, trans.ctypes.data, dfa.n_states, state, out.ctypes.data)
        if rc < 0:
            raise ValueError("automaton state out of range")
        return out.astype(bool)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.artb_tm_destroy(h)


class GrammarState:
    """Cursor of one request: the automaton state after the tokens emitted so far."""

    def __init__(self, dfa: ByteDFA, masker: TokenMasker):
        self.dfa, self.masker, self.state = dfa, masker, 0
        self.failed = False

    def allowed(self) -> np.ndarray:
        """Bool mask over token ids for the next token (only the end-of-sequence token once nothing can follow)."""
        if self.failed:
            m = np.zeros(self.masker.n, dtype=bool)
            if self.masker.eos is not None:
                m[self.masker.eos] = True
            return m
        return self.masker.mask(self.dfa, self.state)

    def advance(self, token_id: int) -> None:
        if token_id == self.masker.eos or self.failed:
            return
        data = self.masker.vocab[token_id] if 0 <= token_id < self.masker.n else b""
        nxt = self.dfa.walk(self.state, data) if data else -1
        if nxt < 0:
            self.failed = True       # a token outside the mask was forced on the sequence: stop constraining
        else:
            self.state = nxt

    @property
    def complete(self) -> bool:
        return not self.failed and bool(self.dfa.accepting[self.state])

    @property
    def exhausted(self) -> bool:
        """Accepting and nothing can follow: the completion is finished whatever the model says."""
        return self.complete and not (self.dfa.trans[self.state] >= 0).any()


class AllowedSet:
    """A fixed set of token ids with the interface of :class:`GrammarState` (``allowed_token_ids`` of a request)."""

    failed = False
    complete = True
    exhausted = False

    def __init__(self, token_ids):
        self.ids = sorted({int(t) for t in token_ids if int(t) >= 0})
        if not self.ids:
            raise ValueError("allowed_token_ids is empty")
        self._mask = np.zeros(self.ids[-1] + 1, dtype=bool)
        self._mask[self.ids] = True

    def allowed(self) -> np.ndarray:
        return self._mask

    def advance(self, token_id: int) -> None:
        pass


_compiled: dict[str, ByteDFA] = {}


def compile_cached(pattern: str) -> ByteDFA:
    dfa = _compiled.get(pattern)
    if dfa is None:
        if len(_compiled) > 256:
            _compiled.clear()
        dfa = _compiled[pattern] = compile_regex(pattern)
    return dfa


def _bench(n_tokens: int = 151_936, seed: int = 0) -> dict:
    """Host-side cost of structured outputs on a synthetic vocabulary of the size of Qwen2.5's: automaton build, trie
    build, and allowed-token masks per automaton state (native walk and its Python twin)."""
    import random
    import string
    import time

    rng = random.Random(seed)
    vocab = [bytes([i]) for i in range(256)]
    chars = string.ascii_letters + string.digits + ' {}[]":,.-_\n'
    while len(vocab) < n_tokens - 1:
        vocab.append("".join(rng.choice(chars) for _ in range(rng.randint(2, 9))).encode())
    vocab.append(b"")
    schema = {"type": "object", "properties": {"name": {"type": "string"}, "age": {"type": "integer"},
                                               "tags": {"type": "array", "items": {"type": "string"}, "maxItems": 4},
                                               "kind": {"enum": ["a", "b", "c"]}}, "required": ["name", "age"]}
    t0 = time.perf_counter()
    dfa = compile_regex(schema_to_regex(schema))
    t_dfa = time.perf_counter() - t0
    from ..ops import _lib

    _lib.runtime()                       # load the library (and what it imports) outside the timed part
    t0 = time.perf_counter()
    native = TokenMasker(vocab, len(vocab) - 1)
    t_trie = time.perf_counter() - t0
    if native._native is None:
        raise SystemExit("the runtime library is not built: python -m art_b200.build")
    plain = TokenMasker(vocab, len(vocab) - 1, use_native=False)
    plain._py_trie()
    states = list(range(dfa.n_states))
    t0 = time.perf_counter()
    counts = [int(native.mask(dfa, s).sum()) for s in states]
    t_native = time.perf_counter() - t0
    widest = max(states, key=lambda s: counts[s])
    native._cache.clear()
    t0 = time.perf_counter()
    native.mask(dfa, widest)
    t_widest = time.perf_counter() - t0
    sample = states[:: max(1, len(states) // 12)]
    t0 = time.perf_counter()
    for s in sample:
        assert int(plain.mask(dfa, s).sum()) == counts[s]
    t_py = time.perf_counter() - t0
    return {"op": "token_mask", "vocabulary": len(vocab), "automaton_states": dfa.n_states,
            "automaton_build_ms": round(t_dfa * 1e3, 1), "trie_build_ms": round(t_trie * 1e3, 1),
            "native_ms_per_state": round(t_native / len(states) * 1e3, 3),
            "native_ms_widest_state": round(t_widest * 1e3, 3), "python_ms_per_state": round(t_py / len(sample) * 1e3, 1),
            "allowed_tokens_min_max": [min(counts), max(counts)]}


if __name__ == "__main__":
    print(json.dumps(_bench()))
