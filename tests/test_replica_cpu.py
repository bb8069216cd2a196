"""Lockstep control of a multi-rank engine replica, on CPU: gloo ranks, reference runner."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys, threading, time, torch, torch.distributed as dist
sys.path.insert(0, os.environ["ARTB_ROOT"])
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
from art_b200.engine.engine import SamplingParams
from art_b200.engine.kv_cache import BlockManager
from art_b200.engine.replica import ReplicaEngine
from art_b200.engine.runner import ReferenceRunner
from art_b200.models.config import PRESETS
from art_b200.models.weights import LoraConfig, init_base_weights, init_lora

cfg = PRESETS["tiny"]
base = init_base_weights(cfg, seed=0)
eng = ReplicaEngine(ReferenceRunner(cfg, base, LoraConfig(), max_loras=2), BlockManager(64, 4, True),
                    ctrl_group=dist.group.WORLD, eos_token_id=None, max_loras=2, num_scheduler_steps=4, keepalive_s=0.2)
out = None
if rank == 0:
    lora = init_lora(cfg, LoraConfig())
    g = torch.Generator().manual_seed(3)
    for k in lora:
        if "lora_B" in k: lora[k] = torch.randn(lora[k].shape, generator=g) * 0.5
    assert eng.set_adapter("m", lora) == 0
    seqs = [eng.add_request([1, 2, 3, 4, 5], SamplingParams(max_tokens=6, temperature=0.0)),
            eng.add_request([9, 8, 7], SamplingParams(max_tokens=9, temperature=1.1), "m"),
            eng.add_request([4, 4, 4, 4], SamplingParams(max_tokens=50, temperature=0.8, top_k=5))]
    n = 0
    while not (seqs[0].finished and seqs[1].finished):
        eng.step(); n += 1
        if n == 2: eng.abort(seqs[2])            # the long request is cancelled on every rank at the same step
    while not seqs[2].finished: eng.step()
    assert seqs[2].finish_reason == "abort" and len(seqs[2].output_ids) < 50
    time.sleep(0.5); eng.step()                  # idle: a keep-alive tick, nothing to do
    eng.start()                                  # now with the background stepping thread
    s4 = eng.add_request([1, 2, 3, 4, 5], SamplingParams(max_tokens=6, temperature=0.0))
    assert s4.done_event.wait(60)
    assert s4.output_ids == seqs[0].output_ids   # prefix-cached, deterministic
    eng.reset_prefix_cache()
    eng.shutdown()
    out = [s.output_ids for s in seqs + [s4]]
else:
    try:
        eng.add_request([1], SamplingParams()); raise SystemExit("followers must refuse requests")
    except RuntimeError:
        pass
    eng.follow()
    out = [eng._seq_of[r].output_ids for r in sorted(eng._seq_of)]
    assert "m" in eng.adapters
allout = [None] * world
dist.all_gather_object(allout, out)
assert all(o == allout[0] for o in allout), allout
assert len(allout[0][0]) == 6 and len(allout[0][1]) == 9
if rank == 0: print("REPLICA_OK", allout[0])
dist.destroy_process_group()
'''


def test_replica_engine_keeps_ranks_in_lockstep(tmp_path):
    script = tmp_path / "replica_worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, ARTB_ROOT=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29631", str(script)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    print(res.stdout[-3000:], res.stderr[-6000:])
    assert res.returncode == 0 and "REPLICA_OK" in res.stdout
