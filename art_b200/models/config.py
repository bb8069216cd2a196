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
    # RoPE frequency scaling as in a Hugging Face config.json: None, or {"rope_type": "linear" | "llama3" | "yarn", ...}
    rope_scaling: dict | None = None

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

    # -- rotary embedding ---------------------------------------------------------------------
    @property
    def rope_type(self) -> str:
        rs = self.rope_scaling or {}
        return str(rs.get("rope_type") or rs.get("type") or "default")

    def rope_inv_freq(self) -> tuple[list[float], float]:
        """``(inverse frequencies [head_dim / 2], attention scale)`` of the rotary embedding.  The angle of pair ``i``
        at position ``p`` is ``p * inv_freq[i]``; cos and sin are multiplied by the attention scale (1 except for
        YaRN).  Covers the unscaled rotation and the ``linear``, ``llama3`` and ``yarn`` variants of Hugging Face
        configurations (same formulas as ``transformers.modeling_rope_utils``)."""
        import math

        hd, base = self.head_dim, float(self.rope_theta)
        rs = dict(self.rope_scaling or {})
        kind = self.rope_type
        inv = [base ** (-(2.0 * i) / hd) for i in range(hd // 2)]
        if kind == "default":
            return inv, 1.0
        factor = float(rs.get("factor", 1.0))
        if kind == "linear":
            return [f / factor for f in inv], 1.0
        if kind == "llama3":
            low, high = float(rs.get("low_freq_factor", 1.0)), float(rs.get("high_freq_factor", 4.0))
            old_len = float(rs.get("original_max_position_embeddings", 8192))
            low_wavelen, high_wavelen = old_len / low, old_len / high
            out = []
            for f in inv:
                wavelen = 2.0 * math.pi / f
                if wavelen > low_wavelen:
                    out.append(f / factor)
                elif wavelen < high_wavelen:
                    out.append(f)
                else:
                    smooth = (old_len / wavelen - low) / (high - low)
                    out.append((1.0 - smooth) * f / factor + smooth * f)
            return out, 1.0
        if kind == "yarn":
            old_len = float(rs.get("original_max_position_embeddings") or self.max_position_embeddings)
            if rs.get("original_max_position_embeddings"):
                factor = float(rs.get("factor", self.max_position_embeddings / old_len))
            beta_fast, beta_slow = float(rs.get("beta_fast") or 32.0), float(rs.get("beta_slow") or 1.0)
            mscale, mscale_all = rs.get("mscale"), rs.get("mscale_all_dim")

            def get_mscale(scale: float, m: float = 1.0) -> float:
                return 1.0 if scale <= 1.0 else 0.1 * m * math.log(scale) + 1.0

            att = rs.get("attention_factor")
            if att is None:
                att = (get_mscale(factor, float(mscale)) / get_mscale(factor, float(mscale_all))
                       if mscale and mscale_all else get_mscale(factor))

            def correction_dim(rot: float) -> float:
                return hd * math.log(old_len / (rot * 2.0 * math.pi)) / (2.0 * math.log(base))

            lo, hi = correction_dim(beta_fast), correction_dim(beta_slow)
            if rs.get("truncate", True):
                lo, hi = math.floor(lo), math.ceil(hi)
            lo, hi = max(lo, 0), min(hi, hd - 1)
            if lo == hi:
                hi += 0.001
            out = []
            for i, f in enumerate(inv):
                ramp = min(1.0, max(0.0, (i - lo) / (hi - lo)))
                extrap = 1.0 - ramp                       # 1: keep the frequency, 0: interpolate (divide by factor)
                out.append(f / factor * (1.0 - extrap) + f * extrap)
            return out, float(att)
        raise ValueError(f"rope scaling of type {kind!r} is not supported (supported: linear, llama3, yarn)")

    # -- what this code base computes, and what it refuses -------------------------------------------
    SUPPORTED_MODEL_TYPES = ("qwen2", "qwen3", "qwen3_moe", "llama", "mistral")

    @staticmethod
    def check_hf_dict(d: dict) -> None:
        """Raises for a Hugging Face configuration whose forward pass differs from what the kernels compute, instead
        of training or serving the checkpoint with silently different numerics."""
        mt = d.get("model_type", "qwen2")
        if mt not in ModelConfig.SUPPORTED_MODEL_TYPES:
            raise ValueError(f"model_type {mt!r} is not supported (supported: {', '.join(ModelConfig.SUPPORTED_MODEL_TYPES)})")
        act = d.get("hidden_act", "silu")
        if act not in ("silu", "swish"):
            raise ValueError(f"hidden_act {act!r} is not supported: the MLP kernels compute SwiGLU")
        if d.get("mlp_bias"):
            raise ValueError("mlp_bias is not supported")
        if mt in ("llama", "mistral") and d.get("attention_bias"):
            raise ValueError("attention_bias on all four projections (o_proj included) is not supported")
        window = d.get("sliding_window")
        if window and d.get("use_sliding_window", mt == "mistral") and window < int(d.get("max_position_embeddings", 0) or 0):
            raise ValueError(f"sliding-window attention (window {window}) is not supported")
        if mt == "qwen3_moe" and (d.get("mlp_only_layers") or int(d.get("decoder_sparse_step") or 1) != 1):
            raise ValueError("sparse models with dense layers in between (mlp_only_layers, decoder_sparse_step != 1) are not supported")
        for k in ("attn_logit_softcapping", "final_logit_softcapping"):
            if d.get(k):
                raise ValueError(f"{k} is not supported")
        rs = d.get("rope_scaling") or d.get("rope_parameters")
        if rs:
            kind = rs.get("rope_type") or rs.get("type") or "default"
            if kind not in ("default", "linear", "llama3", "yarn"):
                raise ValueError(f"rope scaling of type {kind!r} is not supported (supported: linear, llama3, yarn)")

    @classmethod
    def from_hf_dict(cls, d: dict, name: str = "hf") -> "ModelConfig":
        cls.check_hf_dict(d)
        heads = d["num_attention_heads"]
        mt = d.get("model_type", "qwen2")
        rs = d.get("rope_scaling") or d.get("rope_parameters") or None
        if rs and (rs.get("rope_type") or rs.get("type") or "default") == "default":
            rs = None
        theta = d.get("rope_theta") or (d.get("rope_parameters") or {}).get("rope_theta") or 1e4
        return cls(
            name=name, vocab_size=d["vocab_size"], hidden_size=d["hidden_size"], num_layers=d["num_hidden_layers"],
            num_heads=heads, num_kv_heads=d.get("num_key_value_heads", heads),
            head_dim=d.get("head_dim") or d["hidden_size"] // heads,
            intermediate_size=d.get("intermediate_size", 0), rope_theta=float(theta), rope_scaling=dict(rs) if rs else None,
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
                                rope_theta=5e5, rms_norm_eps=1e-5, max_position_embeddings=131072,
                                rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                                              "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}),
    # dense Qwen3 (per-head q/k RMSNorm, no projection bias, head_dim 128 whatever the hidden size)
    "qwen3-0.6b": ModelConfig(name="qwen3-0.6b", family="qwen3", vocab_size=151936, hidden_size=1024, num_layers=28,
                              num_heads=16, num_kv_heads=8, head_dim=128, intermediate_size=3072, qkv_bias=False,
                              qk_norm=True, tie_word_embeddings=True, max_position_embeddings=40960),
    "qwen3-8b": ModelConfig(name="qwen3-8b", family="qwen3", vocab_size=151936, hidden_size=4096, num_layers=36,
                            num_heads=32, num_kv_heads=8, head_dim=128, intermediate_size=12288, qkv_bias=False,
                            qk_norm=True, max_position_embeddings=40960),
    "qwen3-32b": ModelConfig(name="qwen3-32b", family="qwen3", vocab_size=151936, hidden_size=5120, num_layers=64,
                             num_heads=64, num_kv_heads=8, head_dim=128, intermediate_size=25600, qkv_bias=False,
                             qk_norm=True, max_position_embeddings=40960),
    "mistral-7b": ModelConfig(name="mistral-7b", family="mistral", vocab_size=32768, hidden_size=4096, num_layers=32,
                              num_heads=32, num_kv_heads=8, head_dim=128, intermediate_size=14336, qkv_bias=False,
                              rope_theta=1e6, rms_norm_eps=1e-5),
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
