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
                   runs: int = 3, base=None, tp_group=None, prompt_len_max: int = 0) -> dict:
    """Prefill + decode throughput of one engine replica.  ``tp_group``: the replica spans that process group (every
    rank calls this with the same arguments and gets the same numbers).  ``prompt_len_max`` > ``prompt_len`` draws
    prompt lengths uniformly from [prompt_len, prompt_len_max].  The first ``runs - 1`` passes warm every CUDA-graph
    key of the decode loop; the last one is timed with CUDA events."""
    from ..models.weights import LoraConfig, init_base_weights, init_lora
    from ..ops import _lib
    from .engine import Engine, SamplingParams
    from .kv_cache import BlockManager, KVCache
    from .runner import NativeRunner

    dev = torch.device(device)
    tp = 1 if tp_group is None else torch.distributed.get_world_size(tp_group)
    if base is None:
        base = init_base_weights(cfg, seed=0, dtype=torch.bfloat16, device=dev)
    lcfg = LoraConfig()
    bs = 16
    p_hi = max(prompt_len, prompt_len_max)
    nblocks = seqs * ((p_hi + new_tokens) // bs + 2)
    kv = KVCache(cfg.num_layers, nblocks, bs, cfg.num_kv_heads // tp, cfg.head_dim, dev)
    runner = NativeRunner(cfg, lcfg, kv, base=base, max_loras=max(1, loras), device=dev, tp_group=tp_group)
    width = 64
    while width < (p_hi + new_tokens) // bs + 2:
        width *= 2
    runner.table_width = width          # one block-table width for the whole run: no new graph key as contexts grow
    del base
    torch.cuda.empty_cache()
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
    n_sched = eng.n_steps
    # warm passes only have to meet every CUDA-graph key twice (eager, then capture): two full multi-step calls plus
    # the shorter last call of a run, if there is one
    warm_tokens = min(new_tokens, 1 + 2 * n_sched + (new_tokens - 1) % n_sched)
    for run in range(runs):
        timed = run == runs - 1
        n_new = new_tokens if timed else warm_tokens
        if run == runs - 1 and os.environ.get("ARTB_PROFILE_STEP"):
            torch.cuda.synchronize()
            torch.cuda.profiler.start()      # `ncu --profile-from-start off` then sees only the timed run
        reqs = []
        n_prompt = 0
        for i in range(seqs):
            plen = prompt_len if p_hi == prompt_len else int(torch.randint(prompt_len, p_hi + 1, (1,), generator=g))
            n_prompt += plen
            p = torch.randint(0, cfg.vocab_size, (plen,), generator=g).tolist()
            reqs.append(eng.add_request(p, SamplingParams(max_tokens=n_new, temperature=1.0, ignore_eos=True),
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
        if tp > 1:      # device times, maximum over the ranks of the replica
            tt = torch.tensor([t_pre, t_dec], device=dev)
            torch.distributed.all_reduce(tt, op=torch.distributed.ReduceOp.MAX, group=tp_group)
            t_pre, t_dec = float(tt[0]), float(tt[1])
        res = {"model": cfg.name, "tp": tp, "seqs": seqs, "prompt_len": prompt_len if p_hi == prompt_len else [prompt_len, p_hi],
               "new_tokens": new_tokens, "loras": loras,
               "decode_tok_s": round((gen - gen_at_prefill) / t_dec, 1), "prefill_tok_s": round(n_prompt / t_pre, 1),
               "decode_ms_per_step": round(1e3 * t_dec * seqs / max(1, gen - gen_at_prefill), 3),
               "decode_s": round(t_dec, 4), "prefill_s": round(t_pre, 4), "launches": _lib.LAUNCHES - l0}
        for s in reqs:
            eng._release(s)
        eng.running = []
    _lib.check_status(dev)
    runner.close()
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
    ap.add_argument("--prompt-len-max", type=int, default=0, help="draw prompt lengths uniformly up to this")
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel replica over all ranks of a torchrun launch")
    a = ap.parse_args()
    group, dev, rank = None, "cuda", 0
    if a.tp > 1:
        import torch.distributed as dist

        rank, local = int(os.environ["RANK"]), int(os.environ.get("LOCAL_RANK", os.environ["RANK"]))
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        dist.init_process_group("nccl", device_id=dev)
        if dist.get_world_size() != a.tp:
            raise SystemExit("--tp must equal the number of launched ranks")
        group = dist.group.WORLD
    res = measure_decode(PRESETS[a.model], dev, a.seqs, a.prompt_len, a.new_tokens, a.loras, a.runs, tp_group=group,
                         prompt_len_max=a.prompt_len_max)
    if rank == 0:
        print(json.dumps(res))
    if a.tp > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
