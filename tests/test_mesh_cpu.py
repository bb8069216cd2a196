"""Rank layout for combined parallelism: pure arithmetic, then real groups on gloo ranks."""
import os
import subprocess
import sys

import pytest

from art_b200.parallel.mesh import ParallelLayout

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_layout_arithmetic():
    lay = ParallelLayout(8, tp=2)                                   # the TP2 x DP4 benchmark layout
    assert lay.dp == 4 and lay.coords(5) == {"dp": 2, "pp": 0, "cp": 0, "tp": 1}
    assert lay.group_ranks("tp", 5) == [4, 5] and lay.group_ranks("dp", 5) == [1, 3, 5, 7]
    assert lay.data_shard(5) == (2, 4) and lay.data_shard(4) == (2, 4)
    lay = ParallelLayout(8, tp=2, cp=4)                             # the long-context layout: CP4 x TP2
    assert lay.dp == 1 and lay.group_ranks("cp", 3) == [1, 3, 5, 7] and lay.group_ranks("tp", 3) == [2, 3]
    lay = ParallelLayout(16, tp=2, cp=2, pp=2, ep=4)
    assert lay.dp == 2
    for axis in ("dp", "pp", "cp", "tp", "ep"):
        gs = lay.groups()[axis]
        assert sorted(r for g in gs for r in g) == list(range(16))          # a partition of the ranks
        assert all(len(g) == lay.size(axis) if axis != "ep" else len(g) == 4 for g in gs)
        for r in range(16):
            assert r in lay.group_ranks(axis, r)
    for r in range(16):
        assert lay.rank_of(**lay.coords(r)) == r
        assert len({lay.coords(q)["pp"] for q in lay.group_ranks("ep", r)}) == 1   # experts never span stages
    assert ParallelLayout(8, ep=8).group_ranks("ep", 3) == list(range(8))
    with pytest.raises(ValueError):
        ParallelLayout(8, tp=3)
    with pytest.raises(ValueError):
        ParallelLayout(8, pp=2, ep=8)


WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["ARTB_ROOT"])
from art_b200.parallel.mesh import ParallelLayout
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
lay = ParallelLayout(world, tp=2, ep=world)
groups = lay.create_groups()
assert groups["cp"] is None and groups["pp"] is None
for axis in ("tp", "dp", "ep"):
    t = torch.tensor([float(1 << rank)])
    dist.all_reduce(t, group=groups[axis])
    assert int(t.item()) == sum(1 << r for r in lay.group_ranks(axis, rank)), (axis, rank, t)
dist.barrier()
if rank == 0: print("MESH_OK")
dist.destroy_process_group()
'''


def test_groups_on_gloo_ranks(tmp_path):
    script = tmp_path / "mesh_worker.py"
    script.write_text(WORKER)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr",
           "127.0.0.1", "--master-port", "29639", str(script)]
    res = subprocess.run(cmd, env=dict(os.environ, ARTB_ROOT=ROOT), capture_output=True, text=True, timeout=300)
    print(res.stdout[-2000:], res.stderr[-4000:])
    assert res.returncode == 0 and "MESH_OK" in res.stdout
