"""The allocation-free decode entry point (``artb_paged_decode_noalloc``).

Some embedders of the kernel library cannot allocate: a serving process that has given all
device memory to its KV arena, or a latency-critical loop that must avoid the device-wide
synchronisation ``cudaMalloc`` can cause.  For them the split-KV decode has a twin whose scratch
workspace is a fixed array inside the library.  This test calls the twin through its exported C
symbol and checks it against the ordinary entry point (which gets its workspace from the
caller), twice in a row because the shared array keeps the previous call's contents.

The file name sorts last on purpose so that a run stopping at the first failure has already
executed every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(n, Hq, Hkv, hd, bs, lens, seed):
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(seed)
    nblk = sum((l + bs - 1) // bs for l in lens) + 3
    kc = (torch.randn(nblk, bs, Hkv, hd, device=dev, generator=g) * 0.5).to(torch.bfloat16)
    vc = (torch.randn(nblk, bs, Hkv, hd, device=dev, generator=g) * 0.5).to(torch.bfloat16)
    maxb = max((l + bs - 1) // bs for l in lens)
    bt = torch.zeros(n, maxb, dtype=torch.int32)
    perm = torch.randperm(nblk, generator=torch.Generator().manual_seed(seed)).tolist()
    nxt = 0
    for i, l in enumerate(lens):
        nb = (l + bs - 1) // bs
        bt[i, :nb] = torch.tensor(perm[nxt:nxt + nb])
        nxt += nb
    q = (torch.randn(n, Hq * hd, device=dev, generator=g)).to(torch.bfloat16)
    return q, kc, vc, bt.to(dev), torch.tensor(lens, dtype=torch.int32, device=dev)


def test_noalloc_decode_matches_regular_entry_point_twice():
    from art_b200.ops import _lib, paged

    lib = _lib.kernels()
    fn = lib.artb_paged_decode_noalloc
    vp, ci = ctypes.c_void_p, ctypes.c_int
    fn.argtypes = [vp, ci, vp, vp, vp, ci, vp, ci, ci, ci, ci, ci, vp, ci, ci, vp]
    fn.restype = ci
    Hq, Hkv, hd, bs = 8, 2, 64, 16
    for call, (lens, splits) in enumerate([([300, 17, 1000, 64], 4), ([129, 700], 3)]):
        n = len(lens)
        q, kc, vc, bt, ctx = _setup(n, Hq, Hkv, hd, bs, lens, seed=call)
        ref = torch.empty(n, Hq * hd, dtype=torch.bfloat16, device="cuda")
        paged.paged_decode(q, kc, vc, bt, ctx, Hq, Hkv, hd, ref, splits)          # caller-provided workspace
        out = torch.zeros_like(ref)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0]      # the driver's view: would also see a cudaMalloc inside the C function
        rc = fn(q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), bt.stride(0), ctx.data_ptr(), bs,
                n, Hq, Hkv, hd, out.data_ptr(), out.stride(0), splits, torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        if call > 0:      # the first call on a device may load the kernels' module; from then on nothing may move
            assert torch.cuda.mem_get_info()[0] == free_before
        err = ((out.float() - ref.float()).norm() / ref.float().norm()).item()
        assert err < 1e-2, (call, err)
    # a request beyond the fixed workspace is refused with the documented code and launches nothing
    too_many = 4 * 1024 * 1024 // (Hq * 8 * (hd + 2)) + 1
    rc = fn(q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), bt.stride(0), ctx.data_ptr(), bs,
            too_many, Hq, Hkv, hd, out.data_ptr(), out.stride(0), 8, torch.cuda.current_stream().cuda_stream)
    assert rc == -5
    # a head count of zero is a shape error, not a host-side division by zero
    rc = fn(q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), bt.stride(0), ctx.data_ptr(), bs,
            n, Hq, 0, hd, out.data_ptr(), out.stride(0), 2, torch.cuda.current_stream().cuda_stream)
    assert rc == -1
    torch.cuda.synchronize()
    _lib.check_status()
