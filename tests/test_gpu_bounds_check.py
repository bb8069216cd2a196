"""The kernel library built with device-side index checks (``python -m art_b200.build --checked``, loaded with
``ARTB_BOUNDS_CHECK=1``): an index outside its buffer is reported through the status word and the access is skipped.
The out-of-range calls below are only ever made against that library (the worker refuses to run otherwise)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys, torch
sys.path.insert(0, os.environ["ARTB_ROOT"])
from art_b200.ops import _lib, paged, elementwise as ew
assert _lib.bounds_checked(), "this worker must run against the checked library"
assert _lib.kernels()._name.endswith("libartb_kernels_checked.so")
dev = "cuda"
blocks, bs, Hkv, hd = 8, 16, 2, 64
kc = torch.zeros(blocks, bs, Hkv, hd, device=dev, dtype=torch.bfloat16); vc = torch.zeros_like(kc)
M = 6
qkv = torch.randn(M, 4 * hd + 2 * Hkv * hd, device=dev).bfloat16()
slot = torch.tensor([0, 5, blocks * bs + 3, 17, -1, 10 ** 6], dtype=torch.int32, device=dev)     # two slots past the cache
paged.kv_write(qkv, 4 * hd, 4 * hd + Hkv * hd, slot, kc, vc)
torch.cuda.synchronize()
try:
    _lib.check_status(dev); raise SystemExit("no status raised for kv_write")
except _lib.KernelStatusError as e:
    assert e.code == 8, e.code
flat = kc.view(-1, Hkv * hd)
assert torch.equal(flat[5], qkv[1, 4 * hd:4 * hd + Hkv * hd]) and torch.equal(flat[17], qkv[3, 4 * hd:4 * hd + Hkv * hd])
assert int((flat.abs().sum(-1) != 0).sum()) == 3          # rows 0, 5, 17 only: nothing was written anywhere else
_lib.check_status(dev)                                     # the word was reset
# decode attention with a block-table entry past the cache: reported, read as zeros, no fault
n, Hq = 3, 4
q = torch.randn(n, Hq * hd, device=dev).bfloat16()
bt = torch.tensor([[0, 1, 2, 3], [4, 99999, 5, 6], [7, 0, 0, 0]], dtype=torch.int32, device=dev)
ctx = torch.tensor([40, 50, 9], dtype=torch.int32, device=dev)
out = torch.empty(n, Hq * hd, device=dev, dtype=torch.bfloat16)
kc.normal_(); vc.normal_()
paged.paged_decode(q, kc, vc, bt, ctx, Hq, Hkv, hd, out)
torch.cuda.synchronize()
try:
    _lib.check_status(dev); raise SystemExit("no status raised for paged_decode")
except _lib.KernelStatusError as e:
    assert e.code == 8, e.code
assert torch.isfinite(out.float()).all()
# in-range calls raise nothing
table = torch.randn(10, 64, device=dev).bfloat16()
idx = torch.tensor([3, 9, 0], device=dev)
g = ew.gather_rows(table, idx)
assert torch.equal(g, table[idx])
bt[1, 1] = 3
paged.paged_decode(q, kc, vc, bt, ctx, Hq, Hkv, hd, out)
torch.cuda.synchronize(); _lib.check_status(dev)
# a row index past the table: zeros as always, and reported in this build
g = ew.gather_rows(table, torch.tensor([1, 10], device=dev))
torch.cuda.synchronize()
assert float(g[1].abs().sum()) == 0
try:
    _lib.check_status(dev); raise SystemExit("no status raised for gather_rows")
except _lib.KernelStatusError as e:
    assert e.code == 8
print("BOUNDS_CHECK_OK")
'''


def test_checked_library_builds():
    from art_b200 import build as b

    b.build_all(checked=True)
    assert b.CHECKED_KERNEL_LIB.exists() and b.CHECKED_KERNEL_LIB.stat().st_size > 1_000_000


@pytest.mark.gpu
def test_checked_build_reports_bad_indices_and_skips_the_access(tmp_path):
    from art_b200 import build as b

    b.build_all(checked=True)
    script = tmp_path / "bounds_worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, ARTB_ROOT=ROOT, ARTB_BOUNDS_CHECK="1")
    res = subprocess.run([sys.executable, str(script)], env=env, capture_output=True, text=True, timeout=300)
    print(res.stdout[-2000:], res.stderr[-3000:])
    assert res.returncode == 0 and "BOUNDS_CHECK_OK" in res.stdout
