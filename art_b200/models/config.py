"""Architecture descriptions for the supported decoder families.

Dense Qwen2 / Qwen2.5 / Llama-style decoders (RMSNorm, RoPE, GQA, SwiGLU, optional QKV
bias) and Qwen3-MoE-style sparse decoders (per-head q/k RMSNorm, softmax top-k router,
SwiGLU experts).  ``ModelConfig.from_hf_dict`` reads a Hugging Face ``config.json``;
``PRESETS`` holds the shapes used by the benchmarks, instantiated with random weights.
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field


@dataclass
class ModelConfig:
    name: str = "tiny"
    vocab_size: int = 1024
    hidden_size: int = 128
    num_layers: int = 2
    num_heads: int = 4
    num_kv_heads: int = 2
    head_dim: int = 32
    intermediate_size: int = 384
    rope_theta: float = 1e6
    rms_norm_eps: float = 1e-6
    qkv_bias: bool = True
    qk_norm: bool = False          # Qwen3: RMSNorm over head_dim on q and k
    tie_word_embeddings: bool = False
    # MoE (num_experts == 0 -> dense)
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    norm_topk_prob: bool = True
    max_position_embeddings: int = 32768
    family: str = "qwen2"

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def q_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    def to_dict(self) -> dict:
        return asdict(self)

    def num_params(self) -> int:
        d, L = self.hidden_size, self.num_layers
        attn = d * (self.q_size + 2 * self.kv_size) + self.q_size * d
        if self.is_moe:
            mlp = self.num_experts * 3 * d * self.moe_intermediate_size + d * self.num_experts
        else:
            mlp = 3 * d * self.intermediate_size
        emb = self.vocab_size * d * (1 if self.tie_word_embeddings else 2)
        return L * (attn + mlp + 2 * d) + emb + d

    @classmethod
    def from_hf_dict(cls, d: dict, name: str = "hf") -> "ModelConfig":
        heads = d["num_attention_heads"]
        mt = d.get("model_type", "qwen2")
        return cls(
            name=name, vocab_size=d["vocab_size"], hidden_size=d["hidden_size"], num_layers=d["num_hidden_layers"],
            num_heads=heads, num_kv_heads=d.get("num_key_value_heads", heads),
            head_dim=d.get("head_dim") or d["hidden_size"] // heads,
            intermediate_size=d.get("intermediate_size", 0), rope_theta=float(d.get("rope_theta", 1e4)),
            rms_norm_eps=float(d.get("rms_norm_eps", 1e-6)),
            qkv_bias=bool(d.get("attention_bias", mt == "qwen2")), qk_norm=mt.startswith("qwen3"),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            num_experts=int(d.get("num_experts", 0) or d.get("num_local_experts", 0) or 0),
            num_experts_per_tok=int(d.get("num_experts_per_tok", 0) or 0),
            moe_intermediate_size=int(d.get("moe_intermediate_size", 0) or 0),
            norm_topk_prob=bool(d.get("norm_topk_prob", True)),
            max_position_embeddings=int(d.get("max_position_embeddings", 32768)), family=mt,
        )

    @classmethod
    def from_pretrained_dir(cls, path: str) -> "ModelConfig":
        with open(os.path.join(path, "config.json")) as f:
            return cls.from_hf_dict(json.load(f), name=os.path.basename(path.rstrip("/")))


PRESETS: dict[str, ModelConfig] = {
    # CPU oracle configuration: 2 layers, d=128, 4 heads / 2 KV heads, FFN 384, vocab 1024, theta 1e6
    "tiny": ModelConfig(),
    "tiny-moe": ModelConfig(name="tiny-moe", family="qwen3_moe", qkv_bias=False, qk_norm=True, num_experts=8,
                        num_experts_per_tok=2, moe_intermediate_size=64, intermediate_size=0),
    "qwen2.5-0.5b": ModelConfig(name="qwen2.5-0.5b", vocab_size=151936, hidden_size=896, num_layers=24, num_heads=14,
                                num_kv_heads=2, head_dim=64, intermediate_size=4864, tie_word_embeddings=True),
    "qwen2.5-3b": ModelConfig(name="qwen2.5-3b", vocab_size=151936, hidden_size=2048, num_layers=36, num_heads=16,
                              num_kv_heads=2, head_dim=128, intermediate_size=11008, tie_word_embeddings=True),
    "qwen2.5-7b": ModelConfig(name="qwen2.5-7b", vocab_size=152064, hidden_size=3584, num_layers=28, num_heads=28,
                              num_kv_heads=4, head_dim=128, intermediate_size=18944),
    "qwen2.5-14b": ModelConfig(name="qwen2.5-14b", vocab_size=152064, hidden_size=5120, num_layers=48, num_heads=40,
                               num_kv_heads=8, head_dim=128, intermediate_size=13824),
    "qwen2.5-32b": ModelConfig(name="qwen2.5-32b", vocab_size=152064, hidden_size=5120, num_layers=64, num_heads=40,
                               num_kv_heads=8, head_dim=128, intermediate_size=27648),
    "qwen3-30b-a3b": ModelConfig(name="qwen3-30b-a3b", family="qwen3_moe", vocab_size=151936, hidden_size=2048,
                                 num_layers=48, num_heads=32, num_kv_heads=4, head_dim=128, intermediate_size=0,
                                 qkv_bias=False, qk_norm=True, num_experts=128, num_experts_per_tok=8,
                                 moe_intermediate_size=768),
    "llama-3.1-8b": ModelConfig(name="llama-3.1-8b", family="llama", vocab_size=128256, hidden_size=4096, num_layers=32,
                                num_heads=32, num_kv_heads=8, head_dim=128, intermediate_size=14336, qkv_bias=False,
                                rope_theta=5e5, rms_norm_eps=1e-5),
}


def resolve_config(base_model: str, architecture: dict | None = None) -> ModelConfig:
    """``architecture`` dict > local directory with config.json > preset by (fuzzy) name."""
    if architecture:
        return ModelConfig(**architecture)
    if os.path.isdir(base_model) and os.path.exists(os.path.join(base_model, "config.json")):
        return ModelConfig.from_pretrained_dir(base_model)
    key = base_model.lower().removeprefix("random:").split("/")[-1].replace("-instruct", "")
    if key in PRESETS:
        return PRESETS[key]
    for name, cfg in PRESETS.items():
        if name in key:
            return cfg
    raise ValueError(f"unknown base model {base_model!r}: pass init_args['architecture'] or a directory with config.json")
