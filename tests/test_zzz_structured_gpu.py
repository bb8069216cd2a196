"""Structured outputs through the native runner: the allowed-token mask is applied to the fp32 logits of the step on
the device and the restricted sampler draws from what is left.

The file name sorts after the other GPU tests on purpose, like ``test_zz_no_alloc.py``.
"""
import re

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_native_engine_follows_a_guided_regex():
    from art_b200.engine.engine import Engine, SamplingParams
    from art_b200.engine.grammar import TokenMasker, vocabulary_bytes
    from art_b200.engine.kv_cache import BlockManager, KVCache
    from art_b200.engine.runner import NativeRunner
    from art_b200.local.tokenizer import ByteChatTokenizer
    from tests.test_gpu_model import _small_setup

    cfg, base, lcfg, lora = _small_setup()
    tok = ByteChatTokenizer(cfg.vocab_size)
    base_bf = {k: v.to(torch.bfloat16) for k, v in base.items()}
    kv = KVCache(cfg.num_layers, 128, 16, cfg.num_kv_heads, cfg.head_dim, torch.device(DEV))
    eng = Engine(NativeRunner(cfg, lcfg, kv, base=base_bf, max_loras=2, device=DEV), BlockManager(128, 16, True),
                 eos_token_id=tok.eos_token_id, max_loras=2, num_scheduler_steps=4, kv_cache=kv)
    eng.set_adapter("a", {k: v.to(DEV) for k, v in lora.items()})
    eng.token_masker = TokenMasker(vocabulary_bytes(tok), tok.eos_token_id)
    pat = r'\{"move": "(up|down|left|right)", "n": [1-9]\}'
    seqs = [eng.add_request(list(range(5, 30)), SamplingParams(max_tokens=48, guided_regex=pat, seed=i,
                                                                temperature=0.0 if i == 0 else 1.0), "a" if i % 2 else None)
            for i in range(3)]
    free = eng.add_request(list(range(40, 50)), SamplingParams(max_tokens=8, seed=9, ignore_eos=True))
    while not all(s.finished for s in seqs + [free]):
        eng.step()
    for s in seqs:
        text = tok.decode([t for t in s.output_ids if t != tok.eos_token_id])
        assert re.fullmatch(pat, text), text
        assert s.finish_reason == "stop" and all(lp <= 0 and lp == lp for lp in s.logprobs)
    assert len(free.output_ids) == 8
    eng.shutdown()
