"""Rollout throughput probe: ``python -m art_b200.engine.bench_decode --model qwen2.5-7b``.

Fills the engine with ``seqs`` random prompts spread over ``loras`` adapters, lets the scheduler
prefill them, and times the decode phase (CUDA events around it, after one untimed warm-up run).
Used by ``bench.py`` for the rollout half of the headline metric and on its own as the target of
profiler captures of the decode path.
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def measure_decode(cfg, device, seqs: int = 256, prompt_len: int = 512, new_tokens: int = 128, loras: int = 4,
                   runs: int = 3, base=None) -> dict:
    from ..models.weights import LoraConfig, init_base_weights, init_lora
    from ..ops import _lib
    from .engine import Engine, SamplingParams
    from .kv_cache import BlockManager, KVCache
    from .runner import NativeRunner

    dev = torch.device(device)
    if base is None:
        base = init_base_weights(cfg, seed=0, dtype=torch.bfloat16, device=dev)
    lcfg = LoraConfig()
    bs = 16
    nblocks = seqs * ((prompt_len + new_tokens) // bs + 2)
    kv = KVCache(cfg.num_layers, nblocks, bs, cfg.num_kv_heads, cfg.head_dim, dev)
    runner = NativeRunner(cfg, lcfg, kv, base=base, max_loras=max(1, loras), device=dev)
    del base
    eng = Engine(runner, BlockManager(nblocks, bs, False), eos_token_id=None, max_num_seqs=seqs,
                 max_num_batched_tokens=32768, num_scheduler_steps=16, max_loras=max(1, loras), kv_cache=kv)
    for a in range(loras):
        lora = init_lora(cfg, lcfg, seed=a, device=dev)
        g = torch.Generator(device=dev).manual_seed(a)
        for k in lora:
            if "lora_B" in k:
                lora[k] = torch.randn(lora[k].shape, device=dev, generator=g) * 0.01
        eng.set_adapter(f"a{a}", lora)
    g = torch.Generator().manual_seed(0)
    res = {}
    for run in range(runs):
        if run == runs - 1 and os.environ.get("ARTB_PROFILE_STEP"):
            torch.cuda.synchronize()
            torch.cuda.profiler.start()      # `ncu --profile-from-start off` then sees only the timed run
        reqs = []
        for i in range(seqs):
            p = torch.randint(0, cfg.vocab_size, (prompt_len,), generator=g).tolist()
            reqs.append(eng.add_request(p, SamplingParams(max_tokens=new_tokens, temperature=1.0, ignore_eos=True),
                                        f"a{i % loras}" if loras else None))
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        l0 = _lib.LAUNCHES
        e0.record()
        prefilled = False
        gen_at_prefill = 0
        while not all(s.finished for s in reqs):
            eng.step()
            if not prefilled and not eng.waiting:
                e1.record()
                prefilled = True
                gen_at_prefill = sum(len(s.output_ids) for s in reqs)
        e2.record()
        torch.cuda.synchronize()
        gen = sum(len(s.output_ids) for s in reqs)
        t_pre, t_dec = e0.elapsed_time(e1) / 1e3, e1.elapsed_time(e2) / 1e3
        res = {"model": cfg.name, "seqs": seqs, "prompt_len": prompt_len, "new_tokens": new_tokens, "loras": loras,
               "decode_tok_s": round((gen - gen_at_prefill) / t_dec, 1), "prefill_tok_s": round(seqs * prompt_len / t_pre, 1),
               "decode_s": round(t_dec, 4), "prefill_s": round(t_pre, 4), "launches": _lib.LAUNCHES - l0}
        for s in reqs:
            eng._release(s)
        eng.running = []
    _lib.check_status(dev)
    return res


def main() -> None:
    from ..models.config import PRESETS

    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen2.5-7b")
    ap.add_argument("--seqs", type=int, default=256)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--new-tokens", type=int, default=128)
    ap.add_argument("--loras", type=int, default=4)
    ap.add_argument("--runs", type=int, default=3)
    a = ap.parse_args()
    print(json.dumps(measure_decode(PRESETS[a.model], "cuda", a.seqs, a.prompt_len, a.new_tokens, a.loras, a.runs)))


if __name__ == "__main__":
    main()
