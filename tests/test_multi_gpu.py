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


TP_WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["ARTB_ROOT"])
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
from art_b200.parallel.tp import TPContext, unfused_ag_gemm, unfused_gemm_rs
from art_b200.ops import _lib

def rnd(shape, seed, scale=1.0):
    g = torch.Generator(device=dev).manual_seed(seed)
    return (torch.randn(shape, device=dev, generator=g) * scale).to(torch.bfloat16)

def rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-6)).item()

# ---- correctness on small shapes; several calls in a row exercise epoch parity and "done" words
m_seg, K, kt = 256, 320, 64
ctx = TPContext(dev, None, m_seg, k_max=512, n_max=1024, kt=kt)
M = world * m_seg
for it, N in enumerate((512, 264, 1024, 96, 512, 512)):
    x_shard = rnd((m_seg, K), 10 * it + rank)                    # differs per rank
    t_shard = rnd((m_seg, kt), 1000 + 10 * it + rank, 0.3)
    w = rnd((N, K), 77 + it + 31 * rank, 0.05)                   # this rank's column shard
    b2 = rnd((N, kt), 99 + it + 31 * rank, 0.05)
    ctx.ag_input(K).copy_(x_shard)
    ctx.ag_t_input().copy_(t_shard)
    out, x_full, t_full = ctx.ag_gemm(K, w, b2=b2)
    xs = [torch.empty_like(x_shard) for _ in range(world)]; dist.all_gather(xs, x_shard)
    ts = [torch.empty_like(t_shard) for _ in range(world)]; dist.all_gather(ts, t_shard)
    xf, tf = torch.cat(xs), torch.cat(ts)
    ref = xf.float() @ w.float().t() + tf.float() @ b2.float().t()
    torch.cuda.synchronize(); _lib.check_status(dev)
    assert torch.equal(x_full, xf) and torch.equal(t_full, tf), "gathered operands differ"
    e = rel(out, ref)
    assert e < 1e-2, ("ag_gemm", N, e)
# SwiGLU epilogue through the gathered path
N = 512
x_shard = rnd((m_seg, K), 500 + rank); w = rnd((N, K), 600 + rank, 0.05)
ctx.ag_input(K).copy_(x_shard)
h = torch.empty((M, N // 2), dtype=torch.bfloat16, device=dev)
gu, x_full, _ = ctx.ag_gemm(K, w, swiglu_out=h)
g = gu.float().view(M, N // 32, 2, 16)
href = (torch.nn.functional.silu(g[:, :, 0]) * g[:, :, 1]).reshape(M, N // 2)
torch.cuda.synchronize(); _lib.check_status(dev)
assert rel(h, href) < 1e-2

for it, N in enumerate((512, 264, 1024, 96, 512, 512)):
    Kp = 192                                                       # this rank's slice of the reduction dim
    a = rnd((M, Kp), 2000 + 10 * it + rank)
    w = rnd((N, Kp), 3000 + 10 * it + rank, 0.05)
    a2 = rnd((M, kt), 4000 + 10 * it + rank, 0.3)
    b2 = rnd((N, kt), 5000 + it, 0.05)                             # replicated LoRA B
    res = rnd((m_seg, N), 6000 + 10 * it + rank)
    out = ctx.gemm_rs(a, w, a2=a2, b2=b2, residual=res)
    part = a.float() @ w.float().t() + a2.float() @ b2.float().t()
    dist.all_reduce(part)
    ref = part[rank * m_seg:(rank + 1) * m_seg] + res.float()
    torch.cuda.synchronize(); _lib.check_status(dev)
    e = rel(out, ref)
    assert e < 1e-2, ("gemm_rs", N, e)
ctx.close()

# ---- timing at the 7B tensor-parallel shapes (tokens per rank 8192 / world)
def timed(fn, iters=10, warm=3):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(warm): fn()
    dist.barrier(); torch.cuda.synchronize(); e0.record()
    for _ in range(iters): fn()
    e1.record(); torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / iters], device=dev); dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return ms.item()

Mtot, d, ffn = 8192, 3584, 18944
m_seg = Mtot // world
ctx = TPContext(dev, None, m_seg, k_max=d, n_max=d, kt=64)
x_shard = rnd((m_seg, d), 1 + rank)
w_gu = rnd((2 * ffn // world, d), 2 + rank, 0.02)
def fused_ag():
    ctx.ag_input(d).copy_(x_shard)
    ctx.ag_gemm(d, w_gu)
t_fused = timed(fused_ag)
t_unf = timed(lambda: unfused_ag_gemm(x_shard, w_gu))
t_gemm = timed(lambda: torch.cat([x_shard] * world) @ w_gu.t())
fl = 2 * Mtot * (2 * ffn // world) * d
if rank == 0:
    print(f"AG_GEMM_OK world={world} M={Mtot} N={2*ffn//world} K={d} fused_ms={t_fused:.3f} ({fl/t_fused/1e9:.0f} TF/s) "
          f"nccl+cublas_ms={t_unf:.3f} cublas_gemm_only_ms={t_gemm:.3f}")
a = rnd((Mtot, ffn // world), 3 + rank)
w_dn = rnd((d, ffn // world), 4 + rank, 0.02)
res = rnd((m_seg, d), 5 + rank)
t_fused = timed(lambda: ctx.gemm_rs(a, w_dn, residual=res))
t_unf = timed(lambda: unfused_gemm_rs(a, w_dn) + res)
t_gemm = timed(lambda: a @ w_dn.t())
fl = 2 * Mtot * d * (ffn // world)
torch.cuda.synchronize(); _lib.check_status(dev)
if rank == 0:
    print(f"GEMM_RS_OK world={world} M={Mtot} N={d} K={ffn//world} fused_ms={t_fused:.3f} ({fl/t_fused/1e9:.0f} TF/s) "
          f"cublas+nccl_ms={t_unf:.3f} cublas_gemm_only_ms={t_gemm:.3f}")
ctx.close()
dist.destroy_process_group()
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_tp_fused_gemm_collectives(tmp_path):
    world = 1
    while world * 2 <= min(torch.cuda.device_count(), 8):
        world *= 2
    script = tmp_path / "tp_worker.py"
    script.write_text(TP_WORKER)
    env = dict(os.environ, ARTB_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", "29519", str(script)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    print(res.stdout[-3000:], res.stderr[-3000:])
    assert res.returncode == 0 and "AG_GEMM_OK" in res.stdout and "GEMM_RS_OK" in res.stdout
