"""Multi-GPU collectives (needs >= 2 GPUs; spawned as child ranks over NCCL on 127.0.0.1)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["ARTB_ROOT"])
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
from art_b200.parallel.symm_mem import FusedGradAllReduce
from art_b200.ops import _lib
ar = FusedGradAllReduce(dev, world)
for n in (1000, 4 * world * 1000 + 3, 5_000_000):
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    x = torch.randn(n, device=dev, generator=g)
    ref = x.clone()
    dist.all_reduce(ref); ref /= world
    for _ in range(3):          # repeated calls exercise the epoch counters
        y = x.clone()
        ar(y)
    torch.cuda.synchronize(); _lib.check_status(dev)
    err = (y - ref).abs().max().item()
    assert err < 1e-5, (n, err)
e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
y = torch.randn(20_185_088, device=dev)
for _ in range(3): ar(y)
dist.barrier(); torch.cuda.synchronize(); e0.record()
for _ in range(10): ar(y)
e1.record(); torch.cuda.synchronize()
ms = torch.tensor([e0.elapsed_time(e1) / 10], device=dev); dist.all_reduce(ms, op=dist.ReduceOp.MAX)
z = y.clone(); 
for _ in range(3): dist.all_reduce(z)
dist.barrier(); torch.cuda.synchronize(); e0.record()
for _ in range(10): dist.all_reduce(z)
e1.record(); torch.cuda.synchronize()
ms2 = torch.tensor([e0.elapsed_time(e1) / 10], device=dev); dist.all_reduce(ms2, op=dist.ReduceOp.MAX)
if rank == 0: print(f"ALLREDUCE_OK world={world} fused_ms={ms.item():.3f} (incl. 2 staging copies) nccl_ms={ms2.item():.3f} bytes={y.numel()*4}")
dist.destroy_process_group()
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_fused_allreduce_matches_nccl(tmp_path):
    world = min(torch.cuda.device_count(), 8)
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, ARTB_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", "29517", str(script)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    print(res.stdout[-2000:], res.stderr[-3000:])
    assert res.returncode == 0 and "ALLREDUCE_OK" in res.stdout
