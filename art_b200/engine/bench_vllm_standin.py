"""Nearest offline stand-in for the reference's rollout engine: the vLLM that is installed in this image, run on
the same synthetic workload as ``art_b200.engine.bench_decode`` (random-init weights of the same architecture,
token-id prompts, sampling at temperature 1, no stop condition).

The reference serves rollouts with vLLM plus its own patches (src/art/local/vllm.py:22-84, src/art/local/state.py:64-81)
at a pinned version that cannot be installed offline; this script measures the library itself so that the decode
numbers of this repository stand beside something.  It is a baseline only: nothing in the product imports it.

    python -m art_b200.engine.bench_vllm_standin --model qwen2.5-7b --seqs 256 --prompt-len 512 --new-tokens 128

Decode throughput is derived like this: one timed ``generate`` of ``new_tokens`` tokens per sequence and one of a
single token per sequence (prefill + first sample); the difference is the time of ``new_tokens - 1`` decode steps
for all sequences.  Wall-clock timing around blocking library calls (the library synchronises before it returns).
"""
from __future__ import annotations

import argparse
import json
import os
import tempfile
import time


def write_model_dir(cfg, path: str) -> None:
    """A Hugging Face style directory with only a ``config.json`` (weights are drawn by ``load_format="dummy"``)."""
    d = {
        "architectures": ["Qwen3ForCausalLM" if cfg.qk_norm else "Qwen2ForCausalLM"],
        "model_type": "qwen3" if cfg.qk_norm else "qwen2",
        "hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size,
        "num_hidden_layers": cfg.num_layers, "num_attention_heads": cfg.num_heads,
        "num_key_value_heads": cfg.num_kv_heads, "head_dim": cfg.head_dim, "vocab_size": cfg.vocab_size,
        "rms_norm_eps": cfg.rms_norm_eps, "rope_theta": cfg.rope_theta, "max_position_embeddings": 32768,
        "hidden_act": "silu", "tie_word_embeddings": bool(cfg.tie_word_embeddings), "torch_dtype": "bfloat16",
        "attention_bias": bool(cfg.qkv_bias), "use_sliding_window": False, "bos_token_id": 1, "eos_token_id": 2,
    }
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(d, f)


def write_adapters(cfg, root: str, n: int, rank: int = 8) -> list[str]:
    """``n`` PEFT adapter directories with random ``lora_B`` (written by this repository's own checkpoint code)."""
    import torch

    from ..models.peft_io import save_adapter
    from ..models.weights import LoraConfig, init_lora

    out = []
    lcfg = LoraConfig(r=rank, alpha=2 * rank)
    for a in range(n):
        lora = init_lora(cfg, lcfg, seed=a, device="cpu")
        g = torch.Generator().manual_seed(a)
        for k in lora:
            if "lora_B" in k:
                lora[k] = torch.randn(lora[k].shape, generator=g) * 0.01
        path = os.path.join(root, f"adapter{a}")
        save_adapter(path, lora, lcfg, root)
        out.append(path)
    return out


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--model", default="qwen2.5-7b")
    ap.add_argument("--seqs", type=int, default=256)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--new-tokens", type=int, default=128)
    ap.add_argument("--loras", type=int, default=0, help="adapters spread over the sequences (0: base model only)")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.85)
    ap.add_argument("--enforce-eager", action="store_true")
    a = ap.parse_args()

    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    os.environ.setdefault("TRANSFORMERS_OFFLINE", "1")
    os.environ.setdefault("VLLM_NO_USAGE_STATS", "1")
    os.environ.setdefault("DO_NOT_TRACK", "1")
    import torch
    import vllm
    from vllm import LLM, SamplingParams

    from ..models.config import PRESETS

    cfg = PRESETS[a.model]
    root = tempfile.mkdtemp(prefix="vllm-standin-")
    write_model_dir(cfg, root)
    kw = {}
    lora_reqs = None
    if a.loras:
        from vllm.lora.request import LoRARequest

        paths = write_adapters(cfg, root, a.loras)
        kw.update(enable_lora=True, max_loras=a.loras, max_lora_rank=8)
        lora_reqs = [LoRARequest(f"a{i % a.loras}", i % a.loras + 1, paths[i % a.loras]) for i in range(a.seqs)]
    t0 = time.perf_counter()
    llm = LLM(model=root, skip_tokenizer_init=True, load_format="dummy", dtype="bfloat16", tensor_parallel_size=a.tp,
              max_model_len=a.prompt_len + a.new_tokens + 16, max_num_seqs=a.seqs, max_num_batched_tokens=32768,
              gpu_memory_utilization=a.gpu_memory_utilization, enforce_eager=a.enforce_eager, seed=0,
              enable_prefix_caching=False, **kw)
    start_s = time.perf_counter() - t0
    g = torch.Generator().manual_seed(0)
    prompts = [{"prompt_token_ids": torch.randint(0, cfg.vocab_size, (a.prompt_len,), generator=g).tolist()}
               for _ in range(a.seqs)]

    def run(n_new: int) -> float:
        sp = SamplingParams(max_tokens=n_new, temperature=1.0, ignore_eos=True, detokenize=False)
        t = time.perf_counter()
        outs = llm.generate(prompts, sp, lora_request=lora_reqs, use_tqdm=False)
        dt = time.perf_counter() - t
        got = sum(len(o.outputs[0].token_ids) for o in outs)
        if got != a.seqs * n_new:
            raise RuntimeError(f"expected {a.seqs * n_new} tokens, got {got}")
        return dt

    run(min(a.new_tokens, 24))          # warm-up: graphs, allocator
    t_first = min(run(1), run(1))
    t_full = run(a.new_tokens)
    decode_s = max(1e-9, t_full - t_first)
    res = {"op": "vllm_standin_decode", "vllm": vllm.__version__, "model": a.model, "tp": a.tp, "seqs": a.seqs,
           "prompt_len": a.prompt_len, "new_tokens": a.new_tokens, "loras": a.loras, "enforce_eager": a.enforce_eager,
           "engine_start_s": round(start_s, 1), "prefill_s": round(t_first, 4), "total_s": round(t_full, 4),
           "prefill_tok_s": round(a.seqs * a.prompt_len / t_first, 1),
           "decode_tok_s": round(a.seqs * (a.new_tokens - 1) / decode_s, 1),
           "decode_ms_per_step": round(decode_s / max(1, a.new_tokens - 1) * 1e3, 3),
           "weights": "load_format=dummy (random)", "timing": "wall clock around LLM.generate"}
    print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
