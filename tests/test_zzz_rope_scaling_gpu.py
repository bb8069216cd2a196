"""Frequency-scaled rotary embeddings (``rope_scaling`` of a Hugging Face configuration) on the device: the table-driven
rotation kernel against fp32 PyTorch, and the native trainer against the autograd reference with a scaled configuration.

The file name sorts after the other GPU tests on purpose, like ``test_zz_no_alloc.py``.
"""
import dataclasses

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"

LLAMA3 = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 8192}
YARN = {"rope_type": "yarn", "factor": 4.0, "original_max_position_embeddings": 32768}


def rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.mark.parametrize("scaling", [LLAMA3, YARN])
def test_rope_table_kernel_matches_pytorch(scaling):
    from art_b200.models.config import ModelConfig
    from art_b200.ops import elementwise as ew

    M, Hq, Hkv, hd = 300, 4, 2, 128
    cfg = ModelConfig(head_dim=hd, rope_theta=5e5, rope_scaling=dict(scaling))
    kw = ew.rope_args(cfg, DEV)
    assert kw["freqs"].shape == (hd // 2,) and kw["freqs"].device.type == "cuda"
    g = torch.Generator(device=DEV).manual_seed(1)
    buf = torch.randn(M, (Hq + 2 * Hkv) * hd, device=DEV, generator=g).to(torch.bfloat16)
    orig = buf.clone()
    pos = torch.randint(0, 30000, (M,), device=DEV, dtype=torch.int32)
    ew.rope_(buf, pos, 0, Hq + Hkv, hd, cfg.rope_theta, **kw)
    n = (Hq + Hkv) * hd
    ref = ew.rope_reference(orig[:, :n].view(M, Hq + Hkv, hd), pos, cfg.rope_theta, **kw).reshape(M, -1)
    assert rel_err(buf[:, :n], ref) < 5e-3
    assert torch.equal(buf[:, n:], orig[:, n:])                                   # v untouched
    plain = ew.rope_reference(orig[:, :n].view(M, Hq + Hkv, hd), pos, cfg.rope_theta).reshape(M, -1)
    assert rel_err(buf[:, :n], plain) > 0.05                                      # and it is not the unscaled rotation
    ew.rope_(buf, pos, 0, Hq + Hkv, hd, cfg.rope_theta, inverse=True, **kw)
    assert rel_err(buf[:, :n], orig[:, :n].float() * kw["mscale"] ** 2) < 1e-2     # transpose of the forward map


def test_native_trainer_follows_the_scaled_rotation():
    from art_b200.models.config import ModelConfig
    from art_b200.models.weights import LoraConfig, init_base_weights, init_lora
    from art_b200.trainer.trainer import TrainHyper, Trainer
    from tests.test_gpu_model import _packed

    cfg = ModelConfig(name="small-scaled", vocab_size=2048, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2,
                      head_dim=64, intermediate_size=512, rope_scaling={"rope_type": "linear", "factor": 16.0})
    base = init_base_weights(cfg, seed=0)
    for k in base:          # sharper attention than a 0.02-std initialisation gives, so that positions matter: on the
        if "q_proj.weight" in k or "k_proj.weight" in k:      # fp32 oracle the gradients of the scaled and the unscaled
            base[k] = base[k] * 4.0                           # model then have a cosine of 0.38
    lcfg = LoraConfig()
    lora = init_lora(cfg, lcfg, seed=1)
    g = torch.Generator().manual_seed(2)
    for k in lora:
        if "lora_B" in k:
            lora[k] = torch.randn(lora[k].shape, generator=g) * 0.02
    packed = _packed(cfg, 2, 256)
    hy = TrainHyper(learning_rate=1e-4, beta=0.0, rows_per_optimizer_step=2)
    ref = Trainer(cfg, base, lcfg, {k: v.clone() for k, v in lora.items()}, device=DEV, impl="reference")
    nat = Trainer(cfg, base, lcfg, {k: v.clone() for k, v in lora.items()}, device=DEV, impl="native")
    unscaled = Trainer(dataclasses.replace(cfg, rope_scaling=None), base, lcfg, {k: v.clone() for k, v in lora.items()},
                       device=DEV, impl="native")
    mr, mn, mu = ref.step(packed, hy), nat.step(packed, hy), unscaled.step(packed, hy)
    assert abs(mr["loss"] - mn["loss"]) < 5e-3 * max(1.0, abs(mr["loss"]))
    cos = torch.nn.functional.cosine_similarity
    assert cos(ref.flat.grads, nat.flat.grads, dim=0) > 0.99
    assert cos(nat.flat.grads, unscaled.flat.grads, dim=0) < 0.8
