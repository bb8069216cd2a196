"""The serving paths that depend on the tokenizer's vocabulary, on a real byte-level BPE tokenizer (trained in the test:
there is no network and no tokenizer file on the machine): byte strings of the vocabulary, structured outputs with
multi-character tokens, incremental detokenisation."""
import asyncio
import json
import random
import re

import httpx
import pytest

tokenizers = pytest.importorskip("tokenizers")

CORPUS = [
    'The quick brown fox jumps over the lazy dog. {"name": "fox", "age": 3, "tags": ["quick", "brown"]}',
    'She said: "héllo wörld", then left.  {"city": "Zürich", "days": 12, "units": "C"}  true false null 0123456789',
    "日本語のテキストも少し。 Numbers: 10 20 30 400 5000; punctuation: , . : ; ! ? [ ] { } \" ' - _",
] * 20


@pytest.fixture(scope="module")
def bpe():
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers
    from transformers import PreTrainedTokenizerFast

    t = Tokenizer(models.BPE())
    t.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    t.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(vocab_size=600, special_tokens=["<|end|>", "<|user|>", "<|assistant|>"],
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    t.train_from_iterator(CORPUS, trainer)
    tok = PreTrainedTokenizerFast(tokenizer_object=t, eos_token="<|end|>")
    tok.chat_template = ("{% for m in messages %}{{ '<|' + m['role'] + '|>' }}{{ m['content'] }}<|end|>{% endfor %}"
                         "{% if add_generation_prompt %}<|assistant|>{% endif %}")
    return tok


def test_vocabulary_bytes_match_what_the_tokenizer_decodes(bpe):
    from art_b200.engine.grammar import vocabulary_bytes

    vb = vocabulary_bytes(bpe)
    assert len(vb) == len(bpe) and vb[bpe.eos_token_id] == b"" and vb[bpe.convert_tokens_to_ids("<|user|>")] == b""
    multi = 0
    for i, raw in enumerate(vb):
        if not raw:
            continue
        multi += len(raw) > 1
        try:
            text = raw.decode("utf-8")
        except UnicodeDecodeError:
            continue                       # a token that ends inside a character has no text of its own
        assert bpe.decode([i]) == text, (i, raw)
    assert multi > 100                     # merges were learnt: most tokens span several bytes
    # a sentence's tokens concatenate to its bytes
    s = 'She said: "héllo", 日本 {"age": 30}'
    assert b"".join(vb[i] for i in bpe.encode(s)) == s.encode("utf-8")


def test_incremental_decoder_on_bpe_tokens(bpe):
    from art_b200.engine.server import IncrementalDecoder

    rng = random.Random(0)
    ids_all = [i for i in range(len(bpe)) if i not in bpe.all_special_ids]
    for _ in range(30):
        ids = [rng.choice(ids_all) for _ in range(60)]
        dec = IncrementalDecoder(bpe)
        for k in range(0, 60, 7):                      # a scheduler step at a time
            dec.extend(ids[k:k + 7])
        assert dec.final() == bpe.decode(ids, skip_special_tokens=True)
    ids = bpe.encode("héllo wörld 日本語 ok")
    dec = IncrementalDecoder(bpe)
    assert "".join(dec.push(t) for t in ids) == "héllo wörld 日本語 ok"


def test_structured_outputs_through_the_server_with_a_bpe_vocabulary(bpe):
    from art_b200.engine.engine import Engine
    from art_b200.engine.kv_cache import BlockManager
    from art_b200.engine.runner import ReferenceRunner
    from art_b200.engine.server import OpenAIServer
    from art_b200.models.config import PRESETS
    from art_b200.models.weights import LoraConfig, init_base_weights

    cfg = PRESETS["tiny"]                  # 1024 embedding rows for a 600-token vocabulary: the rest is never allowed
    eng = Engine(ReferenceRunner(cfg, init_base_weights(cfg, seed=0), LoraConfig(), max_loras=2), BlockManager(512, 4, True),
                 eos_token_id=bpe.eos_token_id, max_loras=2, num_scheduler_steps=4, max_model_len=1024)
    eng.start()
    srv = OpenAIServer(eng, bpe, "tiny-base", api_key=None)
    schema = {"type": "object", "properties": {"name": {"type": "string", "maxLength": 10}, "age": {"type": "integer", "minimum": 0, "maximum": 99},
                                               "ok": {"type": "boolean"}}, "required": ["name", "age", "ok"]}

    async def main():
        async with httpx.AsyncClient(transport=httpx.ASGITransport(app=srv.app), base_url="http://t") as c:
            msgs = [{"role": "user", "content": "who?"}]
            for seed in range(3):
                r = await c.post("/v1/chat/completions", json={"model": "tiny-base", "messages": msgs, "max_tokens": 80,
                                                               "seed": seed, "guided_json": schema})
                assert r.status_code == 200, r.text
                ch = r.json()["choices"][0]
                val = json.loads(ch["message"]["content"])
                assert ch["finish_reason"] == "stop" and isinstance(val["name"], str) and 0 <= val["age"] <= 99 and isinstance(val["ok"], bool)
                toks = [int(e["token"].split(":")[1]) for e in ch["logprobs"]["content"]]
                assert max(len(bpe.decode([t])) for t in toks) > 1            # multi-character tokens were used
            r = await c.post("/v1/chat/completions", json={"model": "tiny-base", "messages": msgs, "max_tokens": 30, "stream": True,
                                                           "guided_regex": r"(true|false|null)( (true|false|null)){3}"})
            text = "".join(ch["delta"].get("content") or "" for l in r.text.splitlines() if l.startswith("data: {")
                           for ch in json.loads(l[6:])["choices"])
            assert re.fullmatch(r"(true|false|null)( (true|false|null)){3}", text), text
    try:
        asyncio.run(main())
    finally:
        eng.shutdown()


def test_training_tokenisation_splices_sampled_ids_with_a_bpe_tokenizer(bpe):
    """The trainer-side tokenisation (chat template, sentinel splice, shared prompt prefix) with a tokenizer library
    that returns the dictionary form from ``apply_chat_template``."""
    import math

    import art_b200 as art
    from art_b200.local.tokenize import tokenize_trajectory_groups
    from tests.test_api_trajectories import make_choice

    def traj(reward, text):
        ids = bpe.encode(text)
        return art.Trajectory(messages_and_choices=[{"role": "user", "content": "who are you?"}, make_choice(ids, text)],
                              reward=reward), ids

    (ta, ids_a), (tb, ids_b) = traj(1.0, "the quick brown fox"), traj(0.0, "a lazy dog")
    a, b = sorted(tokenize_trajectory_groups(bpe, [art.TrajectoryGroup([ta, tb])], False, random.Random(0)),
                  key=lambda r: -r.advantage)
    prompt = bpe.apply_chat_template([{"role": "user", "content": "who are you?"}], add_generation_prompt=True)
    prompt_ids = list(prompt["input_ids"]) if hasattr(prompt, "keys") else list(prompt)
    n = len(prompt_ids)
    assert a.token_ids[:n] == prompt_ids and a.prompt_length == b.prompt_length == n and a.prompt_id == b.prompt_id
    assert a.token_ids[n:n + len(ids_a)] == ids_a and b.token_ids[n:n + len(ids_b)] == ids_b
    assert sum(a.assistant_mask) == len(ids_a) and a.assistant_mask[n:n + len(ids_a)] == [1] * len(ids_a)
    assert a.logprobs[n] == -0.5 and math.isnan(a.logprobs[0])
    assert bpe.decode(a.token_ids).startswith("<|user|>who are you?<|end|><|assistant|>the quick brown fox")


def test_candidates_and_bad_words_are_encoded_without_special_tokens(bpe):
    """A tokenizer whose ``encode`` puts a beginning-of-text token in front (Llama style): the candidates of
    ``guided_choice`` and the ``bad_words`` of a request sit inside a completion and must not get one."""
    from tokenizers import processors

    from art_b200.engine.engine import Engine
    from art_b200.engine.kv_cache import BlockManager
    from art_b200.engine.runner import ReferenceRunner
    from art_b200.engine.server import OpenAIServer
    from art_b200.models.config import PRESETS
    from art_b200.models.weights import LoraConfig, init_base_weights

    bos = bpe.convert_tokens_to_ids("<|user|>")
    old = bpe.backend_tokenizer.post_processor
    bpe.backend_tokenizer.post_processor = processors.TemplateProcessing(single="<|user|> $A", special_tokens=[("<|user|>", bos)])
    try:
        assert bpe.encode("yes")[0] == bos and bpe.encode("yes", add_special_tokens=False)[0] != bos
        cfg = PRESETS["tiny"]
        eng = Engine(ReferenceRunner(cfg, init_base_weights(cfg, seed=0), LoraConfig(), max_loras=2), BlockManager(256, 4, True),
                     eos_token_id=bpe.eos_token_id, max_loras=2, num_scheduler_steps=2, max_model_len=512)
        eng.start()
        srv = OpenAIServer(eng, bpe, "tiny-base", api_key=None)
        assert all(bos not in w for w in srv._bad_words(["fox"]))

        async def main():
            async with httpx.AsyncClient(transport=httpx.ASGITransport(app=srv.app), base_url="http://t") as c:
                r = await c.post("/v1/chat/completions", json={"model": "tiny-base", "messages": [{"role": "user", "content": "ok?"}],
                                                               "guided_choice": ["yes", "no"]})
                ch = r.json()["choices"][0]
                toks = [int(e["token"].split(":")[1]) for e in ch["logprobs"]["content"]]
                assert ch["message"]["content"] in ("yes", "no") and bos not in toks
        try:
            asyncio.run(main())
        finally:
            eng.shutdown()
    finally:
        bpe.backend_tokenizer.post_processor = old


def test_full_loop_from_a_checkpoint_directory_in_hugging_face_layout(bpe, tmp_path):
    """``base_model`` as a local directory: ``config.json``, tokenizer files and ``model.safetensors`` with the usual
    parameter names are read, rollouts go through the tokenizer's own chat template, a training step produces a PEFT
    adapter.  (CPU: the oracle model and runner; what is under test is the loading and the tokenizer path.)"""
    import os

    from safetensors.torch import save_file

    import art_b200 as art
    from art_b200.local import LocalBackend
    from art_b200.models.config import ModelConfig
    from art_b200.models.weights import init_base_weights

    ckpt = tmp_path / "Tiny-Qwen2-Instruct"
    ckpt.mkdir()
    hf = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "vocab_size": 640, "hidden_size": 64,
          "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2, "intermediate_size": 128,
          "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "max_position_embeddings": 4096, "hidden_act": "silu",
          "tie_word_embeddings": False, "sliding_window": 4096, "use_sliding_window": False, "torch_dtype": "bfloat16"}
    (ckpt / "config.json").write_text(json.dumps(hf))
    cfg = ModelConfig.from_pretrained_dir(str(ckpt))
    assert cfg.name == "Tiny-Qwen2-Instruct" and cfg.head_dim == 16 and cfg.qkv_bias
    weights = {k: v.contiguous() for k, v in init_base_weights(cfg, seed=0).items()}
    save_file(weights, str(ckpt / "model.safetensors"))
    bpe.save_pretrained(str(ckpt))
    assert os.path.exists(ckpt / "tokenizer.json")

    async def main():
        backend = LocalBackend(in_process=True, path=str(tmp_path / "art"))
        model = art.TrainableModel(name="agent", project="p", base_model=str(ckpt),
                                   _internal_config={"init_args": {"max_seq_length": 2048},
                                                     "engine_args": {"num_scheduler_steps": 4, "max_model_len": 512}})
        try:
            await model.register(backend)
            client = model.openai_client()

            async def rollout(i):
                messages = [{"role": "user", "content": "say something"}]
                r = await client.chat.completions.create(model=model.get_inference_name(), messages=messages, max_tokens=8, seed=i)
                return art.Trajectory(messages_and_choices=[*messages, r.choices[0]], reward=float(i % 2))

            groups = await art.gather_trajectory_groups([art.TrajectoryGroup(rollout(i) for i in range(4))], pbar_desc=None)
            choice = groups[0].trajectories[0].messages_and_choices[-1]
            ids = [int(t.token.split(":")[1]) for t in choice.logprobs.content]
            assert all(0 <= t < 640 for t in ids)
            assert bpe.decode([t for t in ids if t != bpe.eos_token_id]) == (choice.message.content or "")
            await model.train(groups, config=art.TrainConfig(learning_rate=1e-3))
            assert await model.get_step() == 1
            out = tmp_path / "art" / "p" / "models" / "agent" / "0001"
            cfg_a = json.load(open(out / "adapter_config.json"))
            assert cfg_a["base_model_name_or_path"] == str(ckpt) and os.path.exists(out / "adapter_model.safetensors")
        finally:
            await model.openai_client().close()
            for s in backend._services.values():
                await s.shutdown()
            backend.close()
    asyncio.run(main())
