"""Model configurations read from Hugging Face ``config.json`` dictionaries: rotary-embedding scaling against the
formulas of ``transformers``, and loud refusal of what the kernels do not compute."""
import pytest
import torch

from art_b200.models.config import PRESETS, ModelConfig
from art_b200.models.reference import ReferenceModel, rope_cos_sin
from art_b200.models.weights import init_base_weights

LLAMA3 = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 8192}


def hf_dict(model_type="llama", **over):
    d = {"model_type": model_type, "vocab_size": 1024, "hidden_size": 256, "num_hidden_layers": 2, "num_attention_heads": 4,
         "num_key_value_heads": 2, "intermediate_size": 512, "rope_theta": 500000.0, "rms_norm_eps": 1e-5,
         "max_position_embeddings": 131072, "hidden_act": "silu"}
    d.update(over)
    return d


@pytest.mark.parametrize("kind,scaling", [
    ("llama3", LLAMA3),
    ("linear", {"rope_type": "linear", "factor": 4.0}),
    ("yarn", {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 32768}),
    ("yarn", {"type": "yarn", "factor": 2.0, "original_max_position_embeddings": 65536, "beta_fast": 16, "beta_slow": 2}),
])
def test_rope_scaling_matches_transformers(kind, scaling):
    from transformers import LlamaConfig
    from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS

    hf = LlamaConfig(hidden_size=256, num_attention_heads=4, num_key_value_heads=2, rope_theta=500000.0,
                     rope_scaling=dict(scaling), max_position_embeddings=131072)
    want, want_att = ROPE_INIT_FUNCTIONS[kind](hf, "cpu")
    cfg = ModelConfig.from_hf_dict(hf.to_dict())          # the library's own serialisation of the configuration
    assert cfg.rope_type == kind
    got, att = cfg.rope_inv_freq()
    torch.testing.assert_close(torch.tensor(got), want, rtol=1e-5, atol=0)
    assert att == pytest.approx(want_att)


def test_unscaled_configuration_has_no_table_and_reference_model_follows_the_scaling():
    cfg = ModelConfig.from_hf_dict(hf_dict("qwen2", sliding_window=131072, use_sliding_window=False))
    assert cfg.rope_scaling is None and cfg.rope_type == "default" and cfg.qkv_bias
    inv, att = cfg.rope_inv_freq()
    assert att == 1.0 and inv[0] == 1.0 and len(inv) == cfg.head_dim // 2
    scaled = ModelConfig.from_hf_dict(hf_dict(rope_scaling=LLAMA3))
    pos = torch.arange(0, 20000, 997)
    c0, s0 = rope_cos_sin(pos, scaled.head_dim, scaled.rope_theta)
    c1, s1 = rope_cos_sin(pos, scaled.head_dim, scaled.rope_theta, scaled)
    torch.testing.assert_close(c0[:, :8], c1[:, :8], atol=5e-3, rtol=0)   # short wavelengths are untouched (fp32 angles)
    torch.testing.assert_close(s0[1:, -1] / s1[1:, -1], torch.full((20,), 8.0), rtol=1e-2, atol=0)   # long ones stretched 8x
    # the whole model: different log-probs with and without the scaling at long positions, equal at position 0
    tiny = PRESETS["tiny"]
    import dataclasses
    a = ReferenceModel(tiny, init_base_weights(tiny, seed=0))
    b = ReferenceModel(dataclasses.replace(tiny, rope_scaling={"rope_type": "linear", "factor": 4.0}), a.base)
    tok = torch.randint(0, tiny.vocab_size, (1, 12), generator=torch.Generator().manual_seed(0))
    ids = torch.zeros(1, 12, dtype=torch.long)
    ha, hb = (m.hidden_states(tok, ids, ids, torch.arange(12).view(1, 12) + 4000) for m in (a, b))
    assert (ha - hb).abs().max() > 1e-4
    torch.testing.assert_close(ha[:, 0], hb[:, 0])       # one token attends to itself: rotation cancels


@pytest.mark.parametrize("over,what", [
    ({"model_type": "gemma3_text"}, "model_type"),
    ({"hidden_act": "gelu_pytorch_tanh"}, "hidden_act"),
    ({"mlp_bias": True}, "mlp_bias"),
    ({"attention_bias": True}, "attention_bias"),
    ({"model_type": "mistral", "sliding_window": 4096, "max_position_embeddings": 32768}, "sliding-window"),
    ({"rope_scaling": {"rope_type": "longrope", "factor": 4.0}}, "longrope"),
    ({"final_logit_softcapping": 30.0}, "softcapping"),
    ({"model_type": "qwen3_moe", "num_experts": 8, "num_experts_per_tok": 2, "moe_intermediate_size": 64, "mlp_only_layers": [0]}, "dense layers"),
    ({"model_type": "qwen2_moe"}, "model_type"),
])
def test_configurations_the_kernels_do_not_cover_are_refused(over, what):
    with pytest.raises(ValueError, match=what):
        ModelConfig.from_hf_dict(hf_dict(**over))


def test_mistral_without_window_and_qwen3_are_accepted():
    m = ModelConfig.from_hf_dict(hf_dict("mistral", sliding_window=None))
    assert not m.qkv_bias and not m.qk_norm and m.head_dim == 64
    q = ModelConfig.from_hf_dict(hf_dict("qwen3", head_dim=128, tie_word_embeddings=True))
    assert q.qk_norm and not q.qkv_bias and q.head_dim == 128 and q.tie_word_embeddings
