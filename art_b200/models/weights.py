"""Parameter containers: frozen base weights (HF names) and LoRA adapters (PEFT names).

Base weights are random-initialised (N(0, 0.02), seeded) for benchmark/test models or
loaded from a local Hugging Face directory of ``*.safetensors`` shards.  LoRA adapters
follow the PEFT convention: ``lora_A [r, in]`` Kaiming-uniform, ``lora_B [out, r]`` zeros,
effective update ``(alpha / r) * B @ A`` (``alpha / sqrt(r)`` with ``use_rslora``).
"""
from __future__ import annotations

import glob
import math
import os
from dataclasses import dataclass, field

import torch

from .config import ModelConfig

ATTN_TARGETS = ("q_proj", "k_proj", "v_proj", "o_proj")
MLP_TARGETS = ("gate_proj", "up_proj", "down_proj")


def linear_shapes(cfg: ModelConfig) -> dict[str, tuple[int, int]]:
    """(out_features, in_features) of every per-layer linear that can carry a LoRA."""
    d = cfg.hidden_size
    shapes = {"self_attn.q_proj": (cfg.q_size, d), "self_attn.k_proj": (cfg.kv_size, d),
              "self_attn.v_proj": (cfg.kv_size, d), "self_attn.o_proj": (d, cfg.q_size)}
    if cfg.is_moe:
        f = cfg.moe_intermediate_size
        for e in range(cfg.num_experts):
            shapes[f"mlp.experts.{e}.gate_proj"] = (f, d)
            shapes[f"mlp.experts.{e}.up_proj"] = (f, d)
            shapes[f"mlp.experts.{e}.down_proj"] = (d, f)
    else:
        f = cfg.intermediate_size
        shapes["mlp.gate_proj"] = (f, d)
        shapes["mlp.up_proj"] = (f, d)
        shapes["mlp.down_proj"] = (d, f)
    return shapes


def init_base_weights(cfg: ModelConfig, seed: int = 0, dtype: torch.dtype = torch.float32,
                      device: str | torch.device = "cpu", std: float = 0.02,
                      scale_residual_out: bool = False) -> dict[str, torch.Tensor]:
    """Random base model in HF naming.  Generated layer by layer on ``device``.

    ``scale_residual_out`` draws the projections that write into the residual stream (``o_proj``, ``down_proj``)
    with ``std / sqrt(2 * num_layers)``, the usual depth-scaled initialisation.  Without it the residual of a deep
    random model is dominated by a component common to all tokens, and a random router then sends almost every
    token to the same few experts, which no trained mixture-of-experts model does."""
    g = torch.Generator(device=device).manual_seed(seed)
    out_scale = (2 * cfg.num_layers) ** -0.5 if scale_residual_out else 1.0

    def rnd(*shape: int, scale: float = 1.0) -> torch.Tensor:
        return (torch.randn(*shape, generator=g, device=device, dtype=torch.float32) * (std * scale)).to(dtype)

    w: dict[str, torch.Tensor] = {"model.embed_tokens.weight": rnd(cfg.vocab_size, cfg.hidden_size)}
    d = cfg.hidden_size
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        for name, (o, n) in linear_shapes(cfg).items():
            w[p + name + ".weight"] = rnd(o, n, scale=out_scale if name.endswith(("o_proj", "down_proj")) else 1.0)
        if cfg.qkv_bias:
            for name in ("q_proj", "k_proj", "v_proj"):
                w[p + f"self_attn.{name}.bias"] = rnd(linear_shapes(cfg)[f"self_attn.{name}"][0])
        if cfg.qk_norm:
            w[p + "self_attn.q_norm.weight"] = torch.ones(cfg.head_dim, dtype=dtype, device=device)
            w[p + "self_attn.k_norm.weight"] = torch.ones(cfg.head_dim, dtype=dtype, device=device)
        if cfg.is_moe:
            w[p + "mlp.gate.weight"] = rnd(cfg.num_experts, d)
        w[p + "input_layernorm.weight"] = torch.ones(d, dtype=dtype, device=device)
        w[p + "post_attention_layernorm.weight"] = torch.ones(d, dtype=dtype, device=device)
    w["model.norm.weight"] = torch.ones(d, dtype=dtype, device=device)
    w["lm_head.weight"] = w["model.embed_tokens.weight"] if cfg.tie_word_embeddings else rnd(cfg.vocab_size, d)
    return w


def load_base_weights(path: str, cfg: ModelConfig, dtype: torch.dtype = torch.bfloat16,
                      device: str | torch.device = "cpu") -> dict[str, torch.Tensor]:
    """Read every ``*.safetensors`` shard in ``path`` (HF layout)."""
    from safetensors import safe_open

    w: dict[str, torch.Tensor] = {}
    files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"no safetensors shards under {path}")
    for fpath in files:
        with safe_open(fpath, framework="pt", device=str(device)) as f:
            for k in f.keys():
                w[k] = f.get_tensor(k).to(dtype)
    if "lm_head.weight" not in w:
        w["lm_head.weight"] = w["model.embed_tokens.weight"]
    return w


@dataclass
class LoraConfig:
    r: int = 8
    alpha: float = 16.0
    target_modules: tuple[str, ...] = ATTN_TARGETS + MLP_TARGETS
    use_rslora: bool = False
    dropout: float = 0.0

    @property
    def scale(self) -> float:
        return self.alpha / math.sqrt(self.r) if self.use_rslora else self.alpha / self.r


PEFT_PREFIX = "base_model.model."


def lora_key(layer: int, module: str, which: str) -> str:
    return f"{PEFT_PREFIX}model.layers.{layer}.{module}.lora_{which}.weight"


def init_lora(cfg: ModelConfig, lcfg: LoraConfig, seed: int = 3407, device: str | torch.device = "cpu",
              expert_range: tuple[int, int] | None = None) -> dict[str, torch.Tensor]:
    """fp32 master LoRA parameters in PEFT naming (A: Kaiming-uniform(a=sqrt 5), B: zeros)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    out: dict[str, torch.Tensor] = {}
    for i in range(cfg.num_layers):
        for module, (o, n) in linear_shapes(cfg).items():
            leaf = module.split(".")[-1]
            if leaf not in lcfg.target_modules:
                continue
            if expert_range is not None and ".experts." in module:
                e = int(module.split(".")[2])
                if not (expert_range[0] <= e < expert_range[1]):
                    continue
            bound = 1.0 / math.sqrt(n)  # kaiming_uniform_(a=sqrt(5)) on [r, in]
            a = (torch.rand(lcfg.r, n, generator=g) * 2 - 1) * bound
            out[lora_key(i, module, "A")] = a.to(device)
            out[lora_key(i, module, "B")] = torch.zeros(o, lcfg.r, device=device)
    return out
