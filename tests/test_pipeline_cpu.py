"""Pipeline-parallel schedule and runner on CPU (gloo ranks as stages)."""
import os
import subprocess
import sys

import pytest

from art_b200.parallel.pp import peak_in_flight, schedule_1f1b, split_layers

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_1f1b_order_properties():
    for P in (1, 2, 3, 4):
        for n in (1, 2, 5, 8):
            for s in range(P):
                ops = schedule_1f1b(s, P, n)
                assert [m for k, m in ops if k == "F"] == list(range(n))
                assert [m for k, m in ops if k == "B"] == list(range(n))
                seen = set()
                for k, m in ops:            # a backward never precedes its forward
                    if k == "F":
                        seen.add(m)
                    else:
                        assert m in seen
                assert peak_in_flight(s, P, n) == min(P - s, n)
    assert schedule_1f1b(0, 2, 3) == [("F", 0), ("F", 1), ("B", 0), ("F", 2), ("B", 1), ("B", 2)]
    assert schedule_1f1b(1, 2, 3) == [("F", 0), ("B", 0), ("F", 1), ("B", 1), ("F", 2), ("B", 2)]


def test_split_layers():
    assert [list(r) for r in split_layers(5, 2)] == [[0, 1, 2], [3, 4]]
    assert sum(len(r) for r in split_layers(28, 8)) == 28


WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["ARTB_ROOT"])
from art_b200.parallel.pp import PipelineRunner, split_layers
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
torch.manual_seed(0)
L, d, n_micro, B = 6, 16, 5, 4
layers = [torch.nn.Linear(d, d) for _ in range(L)]          # identical on every rank (same seed)
data = torch.randn(n_micro, B, d)
target = torch.randn(n_micro, B, d)

class ToyStage:
    def __init__(self, ids, last):
        self.mods = [layers[i] for i in ids]; self.last = last; self.saved = {}
    def forward(self, mb, x):
        x = data[mb] if x is None else x.detach().requires_grad_(True)
        y = x
        for m in self.mods: y = torch.tanh(m(y))
        if self.last:
            y = ((y - target[mb]) ** 2).mean() / n_micro
        self.saved[mb] = (x, y)
        return y.detach()
    def backward(self, mb, dy):
        x, y = self.saved.pop(mb)
        y.backward(dy)
        return x.grad if x.requires_grad else None

ids = split_layers(L, world)[rank]
stage = ToyStage(ids, rank == world - 1)
runner = PipelineRunner(stage, None, act_shape=(B, d), act_dtype=torch.float32)
outs = runner.run(n_micro)
assert not stage.saved
# single-process oracle
ref = [torch.nn.Linear(d, d) for _ in range(L)]
for a, b in zip(ref, layers): a.load_state_dict(b.state_dict())
tot = 0
for mb in range(n_micro):
    y = data[mb]
    for m in ref: y = torch.tanh(m(y))
    loss = ((y - target[mb]) ** 2).mean() / n_micro
    loss.backward(); tot += loss.item()
for i in ids:
    assert torch.allclose(layers[i].weight.grad, ref[i].weight.grad, atol=1e-6), i
    assert torch.allclose(layers[i].bias.grad, ref[i].bias.grad, atol=1e-6), i
# forward-only sweep (the reference-policy pass of the KL term): every micro-batch crosses all stages once
def fwd_only(mb, x):
    y = data[mb] if x is None else x
    with torch.no_grad():
        for m in stage.mods: y = torch.tanh(m(y))
    return y
swept = runner.run_forward(n_micro, fwd_only)
if rank == world - 1:
    assert abs(sum(float(o) for o in outs) - tot) < 1e-6
    with torch.no_grad():
        for mb in range(n_micro):
            y = data[mb]
            for m in ref: y = torch.tanh(m(y))
            assert torch.allclose(swept[mb], y, atol=1e-6), mb
    print("PP_OK", world)
else:
    assert swept == []
dist.destroy_process_group()
'''


@pytest.mark.parametrize("world", [2, 3])
def test_pipeline_runner_matches_single_process(tmp_path, world):
    script = tmp_path / "pp_worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, ARTB_ROOT=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29530 + world), str(script)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=120)
    print(res.stdout[-2000:], res.stderr[-3000:])
    assert res.returncode == 0 and f"PP_OK {world}" in res.stdout
