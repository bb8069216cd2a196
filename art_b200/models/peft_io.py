"""PEFT-format LoRA checkpoints: ``adapter_model.safetensors`` + ``adapter_config.json``.

Tensor names follow PEFT's saved-adapter convention
(``base_model.model.model.layers.{i}.self_attn.q_proj.lora_A.weight`` with ``lora_A [r, in]``,
``lora_B [out, r]``; per-expert paths ``...mlp.experts.{e}.gate_proj...`` for MoE), so a step
directory is consumable by any loader of that format; the reference produces the same layout
through ``trainer.save_model`` (``src/art/local/service.py:50-53,150-153``).
"""
from __future__ import annotations

import json
import os

import torch

from .weights import LoraConfig

ADAPTER_WEIGHTS = "adapter_model.safetensors"
ADAPTER_CONFIG = "adapter_config.json"


def adapter_config_dict(lcfg: LoraConfig, base_model: str) -> dict:
    return {
        "peft_type": "LORA", "task_type": "CAUSAL_LM", "base_model_name_or_path": base_model, "r": lcfg.r,
        "lora_alpha": lcfg.alpha, "lora_dropout": lcfg.dropout, "target_modules": sorted(lcfg.target_modules),
        "bias": "none", "fan_in_fan_out": False, "inference_mode": True, "modules_to_save": None,
        "use_rslora": lcfg.use_rslora, "use_dora": False, "rank_pattern": {}, "alpha_pattern": {},
        "init_lora_weights": True, "layers_to_transform": None, "layers_pattern": None, "revision": None,
        "auto_mapping": None, "peft_version": "art-b200",
    }


def save_adapter(directory: str, state: dict[str, torch.Tensor], lcfg: LoraConfig, base_model: str,
                 dtype: torch.dtype = torch.float32) -> None:
    """Write atomically (temp file + rename) so a crashed writer never leaves a truncated checkpoint."""
    from safetensors.torch import save_file

    os.makedirs(directory, exist_ok=True)
    tensors = {k: v.detach().to("cpu", dtype).contiguous() for k, v in state.items()}
    tmp = os.path.join(directory, ADAPTER_WEIGHTS + ".tmp")
    save_file(tensors, tmp, metadata={"format": "pt"})
    os.replace(tmp, os.path.join(directory, ADAPTER_WEIGHTS))
    tmpc = os.path.join(directory, ADAPTER_CONFIG + ".tmp")
    with open(tmpc, "w") as f:
        json.dump(adapter_config_dict(lcfg, base_model), f, indent=2)
    os.replace(tmpc, os.path.join(directory, ADAPTER_CONFIG))


def load_adapter(directory: str, device: str | torch.device = "cpu") -> tuple[dict[str, torch.Tensor], LoraConfig]:
    from safetensors.torch import load_file

    with open(os.path.join(directory, ADAPTER_CONFIG)) as f:
        c = json.load(f)
    lcfg = LoraConfig(r=int(c["r"]), alpha=float(c["lora_alpha"]), target_modules=tuple(c["target_modules"]),
                      use_rslora=bool(c.get("use_rslora", False)), dropout=float(c.get("lora_dropout", 0.0)))
    state = load_file(os.path.join(directory, ADAPTER_WEIGHTS), device=str(device))
    return {k: v.float() for k, v in state.items()}, lcfg


def is_adapter_dir(path: str) -> bool:
    return os.path.exists(os.path.join(path, ADAPTER_WEIGHTS)) and os.path.exists(os.path.join(path, ADAPTER_CONFIG))
