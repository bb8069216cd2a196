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
    # structured outputs: the vocabulary reaches every rank, which then masks the same tokens
    from art_b200.engine.grammar import vocabulary_bytes
    from art_b200.local.tokenizer import ByteChatTokenizer
    tok = ByteChatTokenizer(cfg.vocab_size)
    eng.set_vocabulary(vocabulary_bytes(tok), tok.eos_token_id)
    s5 = eng.add_request([7, 7, 7], SamplingParams(max_tokens=20, temperature=1.0, seed=5, guided_regex="(left|right)-[0-9]{2}"))
    assert s5.done_event.wait(60)
    import re
    assert re.fullmatch("(left|right)-[0-9]{2}", tok.decode(s5.output_ids)), tok.decode(s5.output_ids)
    eng.reset_prefix_cache()
    eng.shutdown()
    out = [s.output_ids for s in seqs + [s4, s5]]
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


FAIL_WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["ARTB_ROOT"])
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
from art_b200.engine.engine import SamplingParams
from art_b200.engine.kv_cache import BlockManager
from art_b200.engine.replica import ReplicaEngine, ReplicaError
from art_b200.engine.runner import ReferenceRunner
from art_b200.models.config import PRESETS
from art_b200.models.weights import LoraConfig, init_base_weights, init_lora

cfg = PRESETS["tiny"]
runner = ReferenceRunner(cfg, init_base_weights(cfg, seed=0), LoraConfig(), max_loras=2)
if rank == 1:                                    # this rank cannot load the second adapter (host-side failure)
    good = runner.set_adapter
    def flaky(slot, state):
        if slot == 1 and state is not None: raise MemoryError("no room for the adapter on this rank")
        return good(slot, state)
    runner.set_adapter = flaky
eng = ReplicaEngine(runner, BlockManager(64, 4, True), ctrl_group=dist.group.WORLD, eos_token_id=None, max_loras=2,
                    num_scheduler_steps=4)
lora = init_lora(cfg, LoraConfig())
seen = None
if rank == 0:
    eng.set_adapter("a", lora)
    s = eng.generate_sync([1, 2, 3], SamplingParams(max_tokens=4, temperature=0.0), "a")
    assert len(s.output_ids) == 4
    try:
        eng.set_adapter("b", lora)
    except ReplicaError as e:
        seen = "leader: " + str(e)
    try:
        eng.add_request([1, 2], SamplingParams())
    except RuntimeError:
        seen += " | refuses new work"
    eng.shutdown()                               # no tick after a failure: nobody is listening any more
else:
    try:
        eng.follow()
    except MemoryError as e:
        seen = "follower: " + str(e)
allseen = [None] * world
dist.all_gather_object(allseen, seen)
assert allseen[0].startswith("leader: 1 other rank") and allseen[0].endswith("refuses new work"), allseen
assert allseen[1].startswith("follower: no room"), allseen
if rank == 0: print("REPLICA_FAILURE_OK", allseen)
dist.destroy_process_group()
'''


def test_replica_failure_reaches_every_rank(tmp_path):
    script = tmp_path / "replica_fail_worker.py"
    script.write_text(FAIL_WORKER)
    env = dict(os.environ, ARTB_ROOT=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29635", str(script)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    print(res.stdout[-3000:], res.stderr[-6000:])
    assert res.returncode == 0 and "REPLICA_FAILURE_OK" in res.stdout


SHARD_WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["ARTB_ROOT"])
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
from art_b200.engine.runner import NativeRunner
from art_b200.models.config import ModelConfig
from art_b200.models.weights import LoraConfig, init_base_weights, init_lora, lora_key

cfg = ModelConfig(name="small", vocab_size=2048, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2,
                  head_dim=64, intermediate_size=512)
base = {k: v.to(torch.bfloat16) for k, v in init_base_weights(cfg, seed=0).items()}
lcfg = LoraConfig()
lora = init_lora(cfg, lcfg)
g = torch.Generator().manual_seed(5)
for k in lora:
    if "lora_B" in k: lora[k] = torch.randn(lora[k].shape, generator=g) * 0.05
full = NativeRunner(cfg, lcfg, None, base=base, max_loras=2, device="cpu")
part = NativeRunner(cfg, lcfg, None, base=base, max_loras=2, device="cpu", tp_group=dist.group.WORLD)
full.set_adapter(1, lora); part.set_adapter(1, lora)
T, r = world, rank
assert (part.cfg.num_heads, part.cfg.num_kv_heads, part.cfg.intermediate_size) == (4 // T, 2 // T, 512 // T)
ql, kl, fl = part.cfg.q_size, part.cfg.kv_size, part.cfg.intermediate_size
q, kv = cfg.q_size, cfg.kv_size
assert torch.equal(part.lm_head, full.lm_head[r * 2048 // T:(r + 1) * 2048 // T]) and part.vocab_offset == r * 2048 // T
for li in range(cfg.num_layers):
    F, P = full.layers[li], part.layers[li]
    rows = torch.cat([torch.arange(r * ql, (r + 1) * ql), q + torch.arange(r * kl, (r + 1) * kl),
                      q + kv + torch.arange(r * kl, (r + 1) * kl)])
    assert torch.equal(P["qkv"].W, F["qkv"].W[rows]) and torch.equal(P["qkv"].bias_ext[:len(rows)], F["qkv"].bias_ext[rows])
    assert torch.equal(P["qkv"].B_all, F["qkv"].B_all[rows]) and torch.equal(P["qkv"].A_all, F["qkv"].A_all)
    assert torch.equal(P["o"].W, F["o"].W[:, r * ql:(r + 1) * ql])
    assert torch.equal(P["o"].A_all, F["o"].A_all[:, r * ql:(r + 1) * ql]) and torch.equal(P["o"].B_all, F["o"].B_all)
    # gate|up rows are interleaved in blocks of 16: block b of this rank is block r * (fl / 16) + b of the full layer
    blocks = torch.arange(r * fl // 16, (r + 1) * fl // 16)
    gu_rows = (blocks.unsqueeze(1) * 32 + torch.arange(32)).reshape(-1)
    assert torch.equal(P["gu"].W, F["gu"].W[gu_rows]) and torch.equal(P["gu"].B_all, F["gu"].B_all[gu_rows])
    assert torch.equal(P["down"].W, F["down"].W[:, r * fl:(r + 1) * fl])
    assert torch.equal(P["down"].A_all, F["down"].A_all[:, r * fl:(r + 1) * fl])
    # row-parallel LoRA needs no exchange: the partial shrink products add up to the full one
    x = torch.randn(3, cfg.q_size, generator=torch.Generator().manual_seed(li)).to(torch.bfloat16)
    t_part = x[:, r * ql:(r + 1) * ql].float() @ P["o"].A_all.float().t()
    dist.all_reduce(t_part)
    assert torch.allclose(t_part, x.float() @ F["o"].A_all.float().t(), atol=1e-3)
dist.barrier()
if rank == 0: print("SHARDS_OK")
dist.destroy_process_group()
'''


def test_tensor_parallel_runner_shards_reassemble(tmp_path):
    script = tmp_path / "shard_worker.py"
    script.write_text(SHARD_WORKER)
    env = dict(os.environ, ARTB_ROOT=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29633", str(script)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    print(res.stdout[-3000:], res.stderr[-6000:])
    assert res.returncode == 0 and "SHARDS_OK" in res.stdout


def test_serve_replica_launcher_answers_http(tmp_path):
    """Two gloo ranks (reference runner): rank 0 serves HTTP over the replica engine, rank 1 follows."""
    import time

    import httpx

    import socket

    with socket.socket() as sk:                             # a port nobody listens on right now
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29637", "-m", "art_b200.engine.serve_replica", "--reference", "--model", "tiny",
           "--host", "127.0.0.1", "--port", str(port), "--num-blocks", "256", "--block-size", "4",
           "--num-scheduler-steps", "2", "--max-model-len", "512"]
    log = open(tmp_path / "serve.log", "w")
    proc = subprocess.Popen(cmd, env=dict(os.environ, PYTHONPATH=ROOT), stdout=log, stderr=subprocess.STDOUT, cwd=ROOT)
    try:
        hdr = {"Authorization": "Bearer default"}
        base = f"http://127.0.0.1:{port}"
        ok = False
        for _ in range(240):
            if proc.poll() is not None:
                break
            try:
                ok = httpx.get(base + "/v1/models", headers=hdr, timeout=2).status_code == 200
            except httpx.HTTPError:
                ok = False
            if ok:
                break
            time.sleep(0.5)
        assert ok, open(tmp_path / "serve.log").read()[-3000:]
        body = {"model": "tiny", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 6, "n": 2, "seed": 3}
        r = httpx.post(base + "/v1/chat/completions", headers=hdr, json=body, timeout=120)
        assert r.status_code == 200, r.text
        d = r.json()
        assert len(d["choices"]) == 2 and d["usage"]["completion_tokens"] >= 2
        again = httpx.post(base + "/v1/chat/completions", headers=hdr, json=body, timeout=120).json()
        pick = lambda x: [[e["token"] for e in c["logprobs"]["content"]] for c in x["choices"]]  # noqa: E731
        assert pick(again) == pick(d)                       # same seed -> same tokens, on a replica too
        g = dict(body, n=1, guided_choice=["yes", "no"], temperature=0)
        r = httpx.post(base + "/v1/chat/completions", headers=hdr, json=g, timeout=120)
        assert r.status_code == 200 and r.json()["choices"][0]["message"]["content"] in ("yes", "no")
        assert proc.poll() is None                          # both ranks still alive after scoring jobs
    finally:
        proc.terminate()
        try:
            proc.wait(timeout=30)
        except subprocess.TimeoutExpired:
            proc.kill()
        log.close()
