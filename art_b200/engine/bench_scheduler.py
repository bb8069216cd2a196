"""Host-side cost of the rollout engine's scheduler: ``python -m art_b200.engine.bench_scheduler``.

The engine runs with a runner that returns tokens at once, so what is measured is admission, block allocation,
per-token bookkeeping and event delivery alone (no GPU, no model).  Compare the tokens per second printed here with the
decode throughput of the device (``engine/bench_decode.py``): the ratio is the share of a decode step the scheduler
can cost at most when it is not overlapped with the device.
"""
from __future__ import annotations

import argparse
import json
import random
import time

from .engine import Engine, SamplingParams
from .kv_cache import BlockManager


class InstantRunner:
    """The runner interface with no work behind it."""

    last_top_logprobs = None

    def prefill(self, seqs):
        return [7] * len(seqs), [-1.0] * len(seqs)

    def decode(self, seqs, n_steps):
        n = len(seqs)
        return [[7] * n for _ in range(n_steps)], [[-1.0] * n for _ in range(n_steps)]

    def set_adapter(self, slot, state):
        pass


def run(seqs: int = 512, prompt_len: int = 1000, new_tokens: int = 1000, scheduler_steps: int = 16,
        prefix_caching: bool = False) -> dict:
    bs = 16
    eng = Engine(InstantRunner(), BlockManager(seqs * ((prompt_len + new_tokens) // bs + 2), bs, prefix_caching),
                 eos_token_id=None, max_num_seqs=seqs, max_num_batched_tokens=32768, num_scheduler_steps=scheduler_steps,
                 max_model_len=prompt_len + new_tokens + 16)
    rng = random.Random(0)
    reqs = [eng.add_request([rng.randrange(1000) for _ in range(prompt_len)],
                            SamplingParams(max_tokens=new_tokens, stream_events=False)) for _ in range(seqs)]
    t0 = time.perf_counter()
    iters = 0
    while not all(s.finished for s in reqs):
        eng.step()
        iters += 1
    dt = time.perf_counter() - t0
    return {"op": "scheduler_only", "seqs": seqs, "prompt_len": prompt_len, "new_tokens": new_tokens,
            "scheduler_steps": scheduler_steps, "prefix_caching": prefix_caching, "seconds": round(dt, 3),
            "iterations": iters, "ms_per_iteration": round(dt / iters * 1e3, 3),
            "us_per_decode_step": round(dt / (iters * scheduler_steps) * 1e6, 1),
            "tokens_per_s": round(seqs * new_tokens / dt)}


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--seqs", type=int, default=512)
    ap.add_argument("--prompt-len", type=int, default=1000)
    ap.add_argument("--new-tokens", type=int, default=1000)
    ap.add_argument("--scheduler-steps", type=int, default=16)
    ap.add_argument("--prefix-caching", action="store_true")
    a = ap.parse_args()
    print(json.dumps(run(a.seqs, a.prompt_len, a.new_tokens, a.scheduler_steps, a.prefix_caching)))


if __name__ == "__main__":
    main()
