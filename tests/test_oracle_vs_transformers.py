"""The fp32 oracle of this repository (``models/reference.py``, which every kernel test is compared with) against the
model definitions of the ``transformers`` library, on tiny random-weight configurations: same parameter names, same
logits.  This pins the architecture semantics (projection biases, rotary embedding and its scalings, per-head q/k
norms, grouped-query attention, SwiGLU, router and expert mixing) to the upstream definition rather than to a
restatement of it."""
import pytest
import torch

from art_b200.models.config import ModelConfig
from art_b200.models.reference import ReferenceModel
from art_b200.models.weights import init_base_weights

transformers = pytest.importorskip("transformers")

LLAMA3 = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 64}


def _pair(hf_config, hf_cls):
    """The library's model and this repository's configuration + weight dictionary, holding the same weights."""
    torch.manual_seed(0)
    hf_config._attn_implementation = "eager"
    model = hf_cls(hf_config).eval().float()
    cfg = ModelConfig.from_hf_dict(hf_config.to_dict(), name="t")
    ours = init_base_weights(cfg, seed=1)
    # give both the same weights: ours -> theirs (same names; std large enough for attention to matter)
    sd = model.state_dict()
    g = torch.Generator().manual_seed(2)
    for k, v in ours.items():
        if v.dim() == 2 and "embed" not in k and "lm_head" not in k:
            ours[k] = v + torch.randn(v.shape, generator=g) * 0.08
        elif "norm" in k:
            ours[k] = 1.0 + torch.randn(v.shape, generator=g) * 0.1
        elif v.dim() == 1:
            ours[k] = torch.randn(v.shape, generator=g) * 0.1
    theirs = {k: ours[k] for k in sd if k in ours}
    for k in sd:             # the library keeps the experts of a layer stacked in memory (per-expert names on disk)
        if k.endswith("mlp.experts.gate_up_proj"):
            p = k[: -len("gate_up_proj")]
            theirs[k] = torch.stack([torch.cat([ours[f"{p}{e}.gate_proj.weight"], ours[f"{p}{e}.up_proj.weight"]], 0)
                                     for e in range(cfg.num_experts)])
        elif k.endswith("mlp.experts.down_proj"):
            p = k[: -len("down_proj")]
            theirs[k] = torch.stack([ours[f"{p}{e}.down_proj.weight"] for e in range(cfg.num_experts)])
    assert set(sd) - set(theirs) <= {"lm_head.weight"}, set(sd) - set(theirs)
    missing = model.load_state_dict(theirs, strict=False)
    assert not missing.unexpected_keys and set(missing.missing_keys) <= {"lm_head.weight"}
    if "lm_head.weight" in missing.missing_keys:
        ours["lm_head.weight"] = ours["model.embed_tokens.weight"]
    return model, cfg, ours, g


def _check(hf_config, hf_cls, positions=None, atol=2e-4):
    model, cfg, ours, g = _pair(hf_config, hf_cls)
    B, S = 2, 24
    tokens = torch.randint(0, cfg.vocab_size, (B, S), generator=g)
    pos = torch.arange(S).expand(B, S) if positions is None else positions
    with torch.no_grad():
        want = model(input_ids=tokens, position_ids=pos).logits
        ref = ReferenceModel(cfg, ours)
        ids = torch.zeros(B, S, dtype=torch.long)            # one group: plain causal attention
        h = ref.hidden_states(tokens, ids, ids, pos, use_lora=False)
        got = h.float() @ ours["lm_head.weight"].float().t()
    assert got.shape == want.shape
    err = (got - want).abs().max().item()
    assert err < atol * max(1.0, want.abs().max().item()), err


def test_qwen2_matches():
    from transformers import Qwen2Config, Qwen2ForCausalLM

    _check(Qwen2Config(vocab_size=300, hidden_size=64, intermediate_size=160, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=2, rope_theta=1e6, rms_norm_eps=1e-6, max_position_embeddings=512,
                       tie_word_embeddings=False), Qwen2ForCausalLM)


def test_qwen3_with_head_norms_and_tied_embeddings_matches():
    from transformers import Qwen3Config, Qwen3ForCausalLM

    _check(Qwen3Config(vocab_size=300, hidden_size=64, intermediate_size=160, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=32, rope_theta=1e6, rms_norm_eps=1e-6, max_position_embeddings=512,
                       tie_word_embeddings=True, attention_bias=False), Qwen3ForCausalLM)


def test_llama_with_llama3_rope_scaling_matches_at_long_positions():
    from transformers import LlamaConfig, LlamaForCausalLM

    pos = (torch.arange(24) * 37 + 500).expand(2, 24)           # far beyond the original 64 positions
    _check(LlamaConfig(vocab_size=300, hidden_size=64, intermediate_size=160, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=2, rope_theta=10000.0, rms_norm_eps=1e-5, max_position_embeddings=4096,
                       rope_scaling=dict(LLAMA3), tie_word_embeddings=False), LlamaForCausalLM, positions=pos)


def test_mistral_matches():
    from transformers import MistralConfig, MistralForCausalLM

    _check(MistralConfig(vocab_size=300, hidden_size=64, intermediate_size=160, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, head_dim=16, rope_theta=1e6, rms_norm_eps=1e-5, max_position_embeddings=512,
                         sliding_window=None, tie_word_embeddings=False), MistralForCausalLM)


def test_qwen3_moe_matches():
    from transformers import Qwen3MoeConfig, Qwen3MoeForCausalLM

    _check(Qwen3MoeConfig(vocab_size=300, hidden_size=64, intermediate_size=160, moe_intermediate_size=48, num_hidden_layers=2,
                          num_attention_heads=4, num_key_value_heads=2, head_dim=32, num_experts=8, num_experts_per_tok=2,
                          norm_topk_prob=True, rope_theta=1e6, rms_norm_eps=1e-6, max_position_embeddings=512,
                          decoder_sparse_step=1, mlp_only_layers=[], tie_word_embeddings=False, attention_bias=False,
                          output_router_logits=False), Qwen3MoeForCausalLM, atol=5e-4)


def test_engine_greedy_decoding_equals_the_librarys_generate():
    """The rollout engine end to end (scheduler, block manager, reference runner) against ``generate`` of the library:
    the same greedy continuation for several prompts batched together."""
    from transformers import Qwen2Config, Qwen2ForCausalLM

    from art_b200.engine.engine import Engine, SamplingParams
    from art_b200.engine.kv_cache import BlockManager
    from art_b200.engine.runner import ReferenceRunner
    from art_b200.models.weights import LoraConfig

    model, cfg, ours, g = _pair(Qwen2Config(vocab_size=300, hidden_size=64, intermediate_size=160, num_hidden_layers=2,
                                            num_attention_heads=4, num_key_value_heads=2, rope_theta=1e6, rms_norm_eps=1e-6,
                                            max_position_embeddings=512, tie_word_embeddings=False), Qwen2ForCausalLM)
    eng = Engine(ReferenceRunner(cfg, ours, LoraConfig(), max_loras=2), BlockManager(256, 4, True), eos_token_id=None,
                 max_loras=2, num_scheduler_steps=4)
    prompts = [torch.randint(0, 300, (n,), generator=g).tolist() for n in (5, 11, 3)]
    seqs = [eng.add_request(p, SamplingParams(max_tokens=10, temperature=0.0)) for p in prompts]
    while not all(s.finished for s in seqs):
        eng.step()
    for p, s in zip(prompts, seqs):
        with torch.no_grad():
            out = model.generate(torch.tensor([p]), max_new_tokens=10, do_sample=False, pad_token_id=0, eos_token_id=None)
        assert s.output_ids == out[0, len(p):].tolist()


def test_lora_adapters_mean_what_merging_them_into_the_weights_means():
    """The PEFT convention: ``W + (alpha / r) * B @ A`` with ``lora_A`` [r, in] and ``lora_B`` [out, r].  The oracle with
    an adapter gives the logits of the library's model with the merged weights."""
    from transformers import Qwen2Config, Qwen2ForCausalLM

    from art_b200.models.weights import LoraConfig, init_lora

    model, cfg, ours, g = _pair(Qwen2Config(vocab_size=300, hidden_size=64, intermediate_size=160, num_hidden_layers=2,
                                            num_attention_heads=4, num_key_value_heads=2, rope_theta=1e6, rms_norm_eps=1e-6,
                                            max_position_embeddings=512, tie_word_embeddings=False), Qwen2ForCausalLM)
    lcfg = LoraConfig(r=4, alpha=16)
    lora = init_lora(cfg, lcfg, seed=3)
    for k in lora:
        lora[k] = torch.randn(lora[k].shape, generator=g) * 0.1
    merged = dict(model.state_dict())
    n = 0
    for k, a in lora.items():
        if ".lora_A." not in k:
            continue
        b = lora[k.replace(".lora_A.", ".lora_B.")]
        name = k.replace("base_model.model.", "", 1).replace(".lora_A.weight", ".weight")
        merged[name] = merged[name] + (lcfg.alpha / lcfg.r) * (b @ a)
        n += 1
    assert n == 2 * 7
    model.load_state_dict(merged)
    tokens = torch.randint(0, 300, (2, 16), generator=g)
    ids = torch.zeros(2, 16, dtype=torch.long)
    with torch.no_grad():
        want = model(input_ids=tokens).logits
        ref = ReferenceModel(cfg, ours, lora, lcfg)
        got = ref.hidden_states(tokens, ids, ids, None, use_lora=True).float() @ ours["lm_head.weight"].float().t()
        base = ref.hidden_states(tokens, ids, ids, None, use_lora=False).float() @ ours["lm_head.weight"].float().t()
    assert (got - want).abs().max() < 2e-4 * want.abs().max() and (base - want).abs().max() > 1e-2
