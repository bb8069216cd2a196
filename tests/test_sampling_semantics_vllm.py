"""Sampling semantics against the inference library the reference serves through (installed in this image; CPU code
paths only, nothing of it is started): penalties and the top-k / top-p restriction mean here what they mean there."""
import pytest
import torch


def _lib():
    try:
        from vllm.model_executor.layers.utils import apply_penalties
        from vllm.v1.sample.ops.topk_topp_sampler import apply_top_k_top_p
    except Exception as e:  # noqa: BLE001 - not installed, or not importable on this machine
        pytest.skip(f"inference library not importable: {type(e).__name__}")
    return apply_penalties, apply_top_k_top_p


def test_penalties_equal_the_librarys():
    apply_penalties, _ = _lib()
    from art_b200.engine.runner import LogitProc
    from art_b200.ops.paged import build_logit_edits, logit_adjust_

    g = torch.Generator().manual_seed(0)
    for trial in range(20):
        V = 50
        rows = []
        for _ in range(3):
            n_prompt, n_out = int(torch.randint(1, 6, (1,), generator=g)), int(torch.randint(0, 7, (1,), generator=g))
            toks = torch.randint(0, V, (n_prompt + n_out,), generator=g).tolist()
            rows.append((n_prompt, toks, float(torch.rand(1, generator=g) * 1.5 + 0.5), float(torch.rand(1, generator=g) - 0.5),
                         float(torch.rand(1, generator=g) - 0.5)))
        logits = torch.randn(3, V, generator=g) * 3
        pad = lambda xs, n: xs + [V] * (n - len(xs))            # noqa: E731 - the library pads with vocab_size
        prompt = torch.tensor([pad(t[:n], 6) for n, t, *_ in rows])
        out = torch.tensor([pad(t[n:], 7) for n, t, *_ in rows])
        want = apply_penalties(logits.clone(), prompt, out, torch.tensor([r[3] for r in rows]), torch.tensor([r[4] for r in rows]),
                               torch.tensor([r[2] for r in rows]))
        procs = [(LogitProc(n, repetition_penalty=rep, presence_penalty=pres, frequency_penalty=freq), toks)
                 for n, toks, rep, pres, freq in rows]
        got = logit_adjust_(logits.clone(), build_logit_edits(procs))
        torch.testing.assert_close(got, want, atol=1e-5, rtol=1e-5)


def test_top_k_top_p_restriction_equals_the_librarys():
    _, apply_top_k_top_p = _lib()
    from art_b200.ops.paged import reference_restrict

    g = torch.Generator().manual_seed(1)
    for trial in range(300):
        V = 64
        x = torch.randn(1, V, generator=g) * 2
        k = int(torch.randint(1, V + 1, (1,), generator=g))
        p = float(torch.rand(1, generator=g) * 0.94 + 0.05)
        want = torch.isfinite(apply_top_k_top_p(x.clone(), torch.tensor([k]), torch.tensor([p]))[0])
        assert torch.equal(reference_restrict(x[0], k, p), want), (trial, k, p)


def test_hermes_tool_calls_are_extracted_like_the_librarys_parser():
    import json

    try:
        from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers
        from transformers import PreTrainedTokenizerFast
        from vllm.tool_parsers.hermes_tool_parser import Hermes2ProToolParser
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"inference library not importable: {type(e).__name__}")
    from art_b200.engine.tool_parser import HermesToolParser

    t = Tokenizer(models.BPE())
    t.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    t.decoder = decoders.ByteLevel()
    t.train_from_iterator(["tool call text"] * 4, trainers.BpeTrainer(
        vocab_size=300, special_tokens=["<|end|>", "<tool_call>", "</tool_call>"], initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))
    theirs = Hermes2ProToolParser(PreTrainedTokenizerFast(tokenizer_object=t, eos_token="<|end|>"))
    ours = HermesToolParser()
    texts = ['I will look.\n<tool_call>\n{"name": "search", "arguments": {"q": "fox", "n": 3}}\n</tool_call>',
             '<tool_call>\n{"name": "a", "arguments": {}}\n</tool_call>\n<tool_call>\n{"name": "b", "arguments": {"x": [1, 2]}}\n</tool_call>',
             'no tools here', '<tool_call>\n{"name": "broken", "arguments": {\n</tool_call>',
             'text <tool_call>{"name": "inline", "arguments": {"k": "v"}}</tool_call>',
             '<tool_call>\n{"name": "unterminated", "arguments": {"a": 1}}']
    for text in texts:
        r = theirs.extract_tool_calls(text, request=None)
        want = (r.content, [(c.function.name, json.loads(c.function.arguments)) for c in r.tool_calls])
        content, calls = ours.extract(text)
        got = (content, [(c["function"]["name"], json.loads(c["function"]["arguments"])) for c in calls])
        assert got == want, text
