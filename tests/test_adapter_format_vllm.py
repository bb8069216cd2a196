"""The adapter checkpoints this repository writes are read by other tools; the reference's consumer is the LoRA loader
of its inference library.  That library is installed here, so its own checkpoint validation is run over an adapter
written by ``models/peft_io.py`` (configuration and tensor names; no GPU, no engine is started)."""
import os

import pytest


def test_inference_library_accepts_the_adapter_directory(tmp_path):
    try:
        from vllm.lora.peft_helper import PEFTHelper
        from vllm.lora.utils import parse_fine_tuned_lora_name
    except Exception as e:  # noqa: BLE001 - not installed, or not importable on this machine
        pytest.skip(f"inference library not importable: {type(e).__name__}")
    from safetensors import safe_open

    from art_b200.models.config import PRESETS
    from art_b200.models.peft_io import save_adapter
    from art_b200.models.weights import LoraConfig, init_lora, linear_shapes

    cfg = PRESETS["tiny"]
    lcfg = LoraConfig(r=8, alpha=16)
    out = str(tmp_path / "0001")
    save_adapter(out, init_lora(cfg, lcfg), lcfg, "Qwen/Qwen2.5-7B-Instruct")
    helper = PEFTHelper.from_local_dir(out, max_position_embeddings=4096)
    assert helper.r == 8 and helper.lora_alpha == 16 and not helper.use_rslora
    assert sorted(helper.target_modules) == sorted(lcfg.target_modules)
    shapes = linear_shapes(cfg)
    seen = set()
    with safe_open(os.path.join(out, "adapter_model.safetensors"), "pt") as f:
        for key in f.keys():
            module, is_a = parse_fine_tuned_lora_name(key)[:2]
            assert module.startswith("model.layers.")
            proj = module.split(".", 3)[3]                   # "self_attn.q_proj", "mlp.down_proj", ...
            n_out, n_in = shapes[proj]
            assert tuple(f.get_tensor(key).shape) == ((8, n_in) if is_a else (n_out, 8)), key
            seen.add((module, is_a))
    assert len(seen) == 2 * cfg.num_layers * len(lcfg.target_modules)
