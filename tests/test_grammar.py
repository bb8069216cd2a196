"""Structured outputs: byte-level regular-expression automata, JSON schema translation, allowed-token masks (native
trie walk against its Python twin) and the engine's constrained decoding."""
import json
import random
import re
import string

import numpy as np
import pytest

from art_b200.engine.grammar import (GrammarState, RegexError, TokenMasker, any_json, compile_regex, schema_to_regex,
                                     vocabulary_bytes)


def test_automaton_agrees_with_the_re_module_on_random_strings():
    rng = random.Random(0)
    patterns = [r"a*b+c?", r"(ab|cd)*e{2,4}", r"[a-c]{0,3}x", r"\d+(\.\d+)?", r"[^abc]+", r'"([^"\\]|\\.)*"',
                r"(foo|bar|baz){1,2}!", r"x{3}", r"(a|b)*abb", r"\w+@\w+\.(com|org)", r"^(?:a|bc)+?$", r"[\d\s-]{2,}", r"a{2,}\.?"]
    alphabet = 'abcdex.0123@"\\!fozr m-'
    for p in patterns:
        dfa = compile_regex(p)
        for _ in range(1500):
            s = "".join(rng.choice(alphabet) for _ in range(rng.randint(0, 8)))
            assert dfa.matches(s) == bool(re.fullmatch(p, s)), (p, s)


def test_automaton_works_on_utf8_bytes():
    dfa = compile_regex(r"[a-zé日]+!")
    assert dfa.matches("é日a!") and not dfa.matches("ü!")
    state = dfa.walk(0, "é".encode()[:1])            # a token may end in the middle of a character
    assert state >= 0 and not dfa.accepting[state]
    assert dfa.walk(state, "é".encode()[1:] + b"!") >= 0
    dot = compile_regex(r"x.y")
    assert dot.matches("x日y") and dot.matches("x y") and not dot.matches("x\ny")
    neg = compile_regex(r'[^"]*')
    assert neg.matches("añb") and not neg.matches('a"b')


@pytest.mark.parametrize("bad", ["(unclosed", "a{3,2}", "*a", "[abc", "(?=x)y", "a{2000}", "\\", r"\bword\b", r"(a)\1"])
def test_bad_expressions_are_reported(bad):
    with pytest.raises(RegexError):
        compile_regex(bad)


SCHEMA = {
    "type": "object",
    "properties": {
        "name": {"type": "string", "minLength": 1, "maxLength": 8},
        "age": {"type": "integer", "minimum": 0, "maximum": 150},
        "score": {"type": "number"},
        "tags": {"type": "array", "items": {"type": "string"}, "minItems": 1, "maxItems": 3},
        "kind": {"enum": ["a", "b", 3, None]},
        "address": {"$ref": "#/$defs/addr"},
        "alt": {"anyOf": [{"type": "boolean"}, {"type": "null"}]},
    },
    "required": ["name", "age"],
    "$defs": {"addr": {"type": "object", "properties": {"zip": {"type": "string", "pattern": "^[0-9]{5}$"}}, "required": ["zip"]}},
}


def test_json_schema_translation_accepts_and_rejects():
    dfa = compile_regex(schema_to_regex(SCHEMA))
    good = [{"name": "x", "age": 3}, {"name": "é\n\"q", "age": 150, "score": -1.5e3, "tags": ["a", "b"], "kind": None},
            {"name": "abcdefgh", "age": 0, "kind": 3, "address": {"zip": "12345"}, "alt": True},
            {"name": "x", "age": 7, "tags": ["a", "b", "c"], "alt": None}]
    for v in good:
        for text in (json.dumps(v, ensure_ascii=False), json.dumps(v, ensure_ascii=False, separators=(",", ":"))):
            assert dfa.matches(text), text
    bad = ['{"age":3}', '{"name":"x"}', '{"name":"","age":3}', '{"name":"abcdefghi","age":3}', '{"name":"x","age":3.5}',
           '{"name":"x","age":-1}', '{"name":"x","age":3,"tags":[]}', '{"name":"x","age":3,"tags":["a","b","c","d"]}',
           '{"name":"x","age":3,"kind":"c"}', '{"name":"x","age":3,"address":{"zip":"1234"}}', '{"age":3,"name":"x"}',
           '{"name":"x","age":3,"extra":1}', '{"name":"x","age":3}  x', '{"name":"x","age":1234}']
    for text in bad:
        assert not dfa.matches(text), text
    # no required property: the empty object and any subset in order
    opt = compile_regex(schema_to_regex({"type": "object", "properties": {"a": {"type": "integer"}, "b": {"type": "boolean"},
                                                                           "c": {"type": "null"}}}))
    for text in ("{}", '{"a":1}', '{"b":true}', '{"c":null}', '{"a":1,"c":null}', '{"a": 1, "b": false, "c": null}'):
        assert opt.matches(text), text
    assert not opt.matches('{"b":true,"a":1}') and not opt.matches('{"a":1,}')
    # free-form values
    free = compile_regex(any_json(2))
    assert free.matches('{"a": [1, 2.5, "x"], "b": {"c": null}}') and not free.matches('{"a": [[[1]]]}')
    assert compile_regex(schema_to_regex({"type": "object"})).matches('{"k": [1, {"z": true}]}')
    with pytest.raises(ValueError):
        schema_to_regex({"$ref": "#/$defs/n", "$defs": {"n": {"type": "object", "properties": {"next": {"$ref": "#/$defs/n"}},
                                                              "required": ["next"]}}})


def _vocab(n=20000, seed=0):
    rng = random.Random(seed)
    vocab = [bytes([i]) for i in range(256)]
    vocab += [w.encode() for w in ('{"', '"}', '":', '": "', '", "', "name", "age", "true", "false", "null", "123", "é", "日本")]
    chars = string.ascii_letters + string.digits + ' {}[]":,.-_'
    while len(vocab) < n:
        vocab.append("".join(rng.choice(chars) for _ in range(rng.randint(2, 7))).encode())
    vocab.append(b"")          # a special token: never allowed
    vocab.append(b"")          # the end-of-sequence token
    return vocab


def test_native_masks_equal_the_python_walk_and_drive_a_valid_completion():
    vocab = _vocab()
    eos = len(vocab) - 1
    native, plain = TokenMasker(vocab, eos), TokenMasker(vocab, eos, use_native=False)
    assert native._native is not None, "the runtime library with the trie walk must be built"
    dfa = compile_regex(schema_to_regex({"type": "object", "properties": {"name": {"type": "string"}, "age": {"type": "integer"}},
                                         "required": ["name", "age"]}))
    for s in range(dfa.n_states):
        a, b = native.mask(dfa, s), plain.mask(dfa, s)
        assert (a == b).all(), s
        assert not a[eos - 1] and a[eos] == bool(dfa.accepting[s])
    rng = random.Random(1)
    for trial in range(20):
        g = GrammarState(dfa, native)
        out = b""
        for _ in range(400):
            ids = np.flatnonzero(g.allowed())
            assert len(ids)
            t = int(rng.choice(ids))
            if t == eos or g.exhausted:
                break
            out += vocab[t]
            g.advance(t)
            if len(out) > 60 and g.complete:
                break
            if len(out) > 60:       # steer to the end: prefer tokens that close the string / the object
                closing = [i for i in ids if vocab[i][:1] in (b'"', b"}", b",", b":") or vocab[i].isdigit()]
                if closing:
                    t2 = int(rng.choice(closing))
                    if t2 != eos:
                        out += vocab[t2]
                        g.advance(t2)
        if g.complete:
            val = json.loads(out)
            assert isinstance(val["name"], str) and isinstance(val["age"], int)
    g = GrammarState(dfa, native)
    g.advance(vocab.index(b"name"))         # a token outside the mask was forced: the cursor stops constraining
    assert g.failed and g.allowed().sum() == 1 and g.allowed()[eos]


def test_vocabulary_bytes_of_byte_level_and_sentencepiece_tokenizers():
    from art_b200.engine.grammar import _gpt2_byte_decoder
    from art_b200.local.tokenizer import ByteChatTokenizer

    tok = ByteChatTokenizer(300)
    vb = vocabulary_bytes(tok)
    assert vb[65] == b"A" and vb[256] == b"" and len(vb) == 300
    enc = {b: c for c, b in _gpt2_byte_decoder().items()}

    class ByteLevel:            # GPT-2 style: bytes shown as printable characters, 'Ġ' for a space
        toks = ["".join(enc[b] for b in s.encode()) for s in (" the", "é", "\n", "a")] + ["<|endoftext|>"]
        all_special_ids = [4]

        def __len__(self):
            return len(self.toks)

        def convert_ids_to_tokens(self, ids):
            return [self.toks[i] for i in ids]

    assert ByteLevel.toks[0] == "Ġthe"
    assert vocabulary_bytes(ByteLevel()) == [b" the", "é".encode(), b"\n", b"a", b""]

    class Sentencepiece:
        toks = ["▁the", "<0x0A>", "é", "<s>"]
        all_special_ids = [3]

        def __len__(self):
            return len(self.toks)

        def convert_ids_to_tokens(self, ids):
            return [self.toks[i] for i in ids]

    assert vocabulary_bytes(Sentencepiece()) == [b" the", b"\n", "é".encode(), b""]


def test_engine_mixes_constrained_and_free_sequences_in_one_batch():
    import torch

    from art_b200.engine.engine import Engine, SamplingParams
    from art_b200.engine.kv_cache import BlockManager
    from art_b200.engine.runner import ReferenceRunner
    from art_b200.local.tokenizer import ByteChatTokenizer
    from art_b200.models.config import PRESETS
    from art_b200.models.weights import LoraConfig, init_base_weights

    cfg = PRESETS["tiny"]
    tok = ByteChatTokenizer(cfg.vocab_size)
    eng = Engine(ReferenceRunner(cfg, init_base_weights(cfg, seed=0), LoraConfig(), max_loras=2), BlockManager(128, 4, True),
                 eos_token_id=tok.eos_token_id, max_loras=2, num_scheduler_steps=4)
    with pytest.raises(ValueError, match="token_masker"):
        eng.add_request([1, 2, 3], SamplingParams(guided_regex="a+"))
    eng.token_masker = TokenMasker(vocabulary_bytes(tok), tok.eos_token_id)
    pat = r"(red|green|blue)( (red|green|blue)){2}\."
    a = eng.add_request([1, 2, 3], SamplingParams(max_tokens=40, guided_regex=pat, seed=1))
    b = eng.add_request([1, 2, 3], SamplingParams(max_tokens=12, seed=1, ignore_eos=True))
    c = eng.add_request([4, 5], SamplingParams(max_tokens=40, guided_regex=r"-?[0-9]{1,3}", temperature=0.0))
    while not (a.finished and b.finished and c.finished):
        eng.step()
    assert re.fullmatch(pat, tok.decode(a.output_ids)) and a.finish_reason == "stop"
    assert len(b.output_ids) == 12 and b.finish_reason == "length"
    text_c = tok.decode([t for t in c.output_ids if t != tok.eos_token_id])
    assert re.fullmatch(r"-?[0-9]{1,3}", text_c) and c.finish_reason == "stop"
    assert all(lp <= 0 and lp == lp for lp in a.logprobs + c.logprobs)
    assert torch.isfinite(torch.tensor(a.logprobs)).all()


def _random_accepted_text(dfa, rng, max_len=400):
    """A random walk through the automaton that ends in an accepting state (None if it runs too long).  Bytes are
    drawn from what the current state allows, preferring printable ASCII so that strings stay short and readable."""
    state, out = 0, bytearray()
    while len(out) < max_len:
        if dfa.accepting[state] and (rng.random() < 0.3 or not (dfa.trans[state] >= 0).any()):
            return bytes(out)
        allowed = np.flatnonzero(dfa.trans[state] >= 0)
        if len(allowed) == 0:
            return bytes(out) if dfa.accepting[state] else None
        closing = [b for b in allowed if b in b'"}],:']
        pick = int(rng.choice(closing)) if closing and rng.random() < 0.35 else int(rng.choice(allowed))
        out.append(pick)
        state = int(dfa.trans[state, pick])
    return None


def test_everything_the_automaton_accepts_satisfies_the_schema():
    """Soundness against an independent validator: random texts drawn from the automaton parse as JSON and validate
    against the schema they were compiled from."""
    jsonschema = pytest.importorskip("jsonschema")
    schemas = [SCHEMA,
               {"type": "array", "items": {"type": "object", "properties": {"id": {"type": "integer", "minimum": 1, "maximum": 500},
                                                                              "tag": {"enum": ["x", "y"]}}, "required": ["id"]},
                "minItems": 1, "maxItems": 3},
               {"type": "object", "properties": {"when": {"type": "string", "format": "date"}, "ratio": {"type": "number"},
                                                 "flags": {"type": "array", "items": {"type": "boolean"}}}, "required": ["when", "ratio"]},
               {"anyOf": [{"type": "string", "maxLength": 5}, {"type": "integer"}, {"type": "null"}]}]
    rng = random.Random(0)
    for schema in schemas:
        dfa = compile_regex(schema_to_regex(schema))
        checked = 0
        for _ in range(400):
            raw = _random_accepted_text(dfa, rng)
            if raw is None:
                continue
            try:
                text = raw.decode("utf-8")
            except UnicodeDecodeError:
                continue                      # a random walk over bytes may stop inside a character
            value = json.loads(text)
            bounded = {k: v for k, v in schema.items()}
            jsonschema.validate(value, bounded, format_checker=None)
            checked += 1
        assert checked > 50, (schema, checked)


def test_instances_of_a_schema_are_accepted_in_compact_and_spaced_form():
    """Completeness on random instances (built by a small generator): what satisfies the schema is accepted as
    ``json.dumps`` writes it, with and without spaces."""
    rng = random.Random(1)
    dfa = compile_regex(schema_to_regex(SCHEMA))
    for _ in range(200):
        inst = {"name": "".join(rng.choice("abcé\"\\ \n") for _ in range(rng.randint(1, 8))), "age": rng.randint(0, 150)}
        if rng.random() < 0.5:
            inst["score"] = rng.choice([0, -1.5, 3.25e10, 7, -2e-3])
        if rng.random() < 0.5:
            inst["tags"] = ["".join(rng.choice("xyz ") for _ in range(rng.randint(0, 4))) for _ in range(rng.randint(1, 3))]
        if rng.random() < 0.5:
            inst["kind"] = rng.choice(["a", "b", 3, None])
        if rng.random() < 0.3:
            inst["address"] = {"zip": "".join(rng.choice("0123456789") for _ in range(5))}
        if rng.random() < 0.3:
            inst["alt"] = rng.choice([True, False, None])
        for text in (json.dumps(inst, ensure_ascii=False), json.dumps(inst, ensure_ascii=False, separators=(",", ":")),
                     json.dumps(inst)):
            assert dfa.matches(text), text


def test_integer_ranges_are_exact():
    from art_b200.engine.grammar import int_range_regex

    rng = random.Random(0)
    for _ in range(120):
        a = rng.randint(-1500, 1500)
        b = a + rng.choice([0, 1, 5, 37, 999, 2600])
        pat = re.compile(int_range_regex(a, b))
        for v in list(range(a - 25, a + 25)) + list(range(b - 25, b + 25)) + [rng.randint(-5000, 5000) for _ in range(40)]:
            assert bool(pat.fullmatch(str(v))) == (a <= v <= b), (a, b, v)
        assert not pat.fullmatch("-0") and not pat.fullmatch("007") and not pat.fullmatch("+1")
    dfa = compile_regex(schema_to_regex({"type": "integer", "minimum": -3, "maximum": 12}))
    assert [v for v in range(-10, 20) if dfa.matches(str(v))] == list(range(-3, 13))
    ex = compile_regex(schema_to_regex({"type": "integer", "exclusiveMinimum": 0, "exclusiveMaximum": 10}))
    assert [v for v in range(-3, 13) if ex.matches(str(v))] == list(range(1, 10))


def test_schemas_written_by_pydantic_models_are_understood():
    """What ``client.beta.chat.completions.parse(response_format=Model)`` sends: ``$defs`` with references, enums,
    bounded integers, ``Optional`` as ``anyOf``, literals, bounded lists, dictionaries as ``additionalProperties``."""
    from enum import Enum
    from typing import Literal, Optional

    from pydantic import BaseModel, Field

    class Color(str, Enum):
        red = "red"
        blue = "blue"

    class Item(BaseModel):
        sku: str = Field(max_length=8)
        qty: int = Field(ge=1, le=20)
        color: Color

    class Order(BaseModel):
        id: int
        items: list[Item] = Field(min_length=1, max_length=2)
        note: Optional[str] = None
        kind: Literal["a", "b"] = "a"
        price: float
        meta: dict[str, int] = {}

    dfa = compile_regex(schema_to_regex(Order.model_json_schema()))
    full = Order(id=5, items=[Item(sku="ab", qty=3, color=Color.red)], note="hi", kind="b", price=2.5, meta={"x": 1})
    short = Order(id=1, items=[Item(sku="z", qty=20, color="blue")] * 2, price=1)
    for o in (full, short):
        for text in (o.model_dump_json(), json.dumps(o.model_dump(mode="json"))):
            assert dfa.matches(text), text
            Order.model_validate_json(text)
    for bad in ('{"id":5,"items":[],"price":1.0}',
                '{"id":5,"items":[{"sku":"a","qty":21,"color":"red"}],"note":null,"kind":"a","price":1.0,"meta":{}}',
                '{"id":5,"items":[{"sku":"a","qty":2,"color":"green"}],"note":null,"kind":"a","price":1.0,"meta":{}}',
                '{"id":5,"items":[{"sku":"a","qty":2,"color":"red"}],"note":null,"kind":"c","price":1.0,"meta":{}}'):
        assert not dfa.matches(bad), bad
