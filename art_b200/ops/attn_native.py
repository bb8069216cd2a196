"""ctypes front-end of the tree-masked flash attention kernels (``csrc/kernels/attn_tree.cu``)."""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass

import torch

from . import _lib

vp, ci = ctypes.c_void_p, ctypes.c_int
_sigs = {
    "artb_attn_tile_states": [vp, vp, vp, ci, ci, vp],
    "artb_attn_tree_fwd": [vp, ci, vp, vp, vp, vp, ci, vp, ci, ci, ci, ci, ci, vp],
    "artb_attn_tree_bwd": [vp, ci, vp, vp, ci, vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, vp],
    "artb_attn_tc_fwd": [vp, ci, vp, vp, vp, vp, vp, ci, vp, ci, ci, ci, ci, vp, vp],
    "artb_attn_tc_bwd": [vp, ci, vp, vp, ci, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, vp, vp],
}
# forward on tcgen05 / TMEM when the shape allows it (head dim 128, rows a multiple of 128 tokens)
USE_TC = os.environ.get("ARTB_ATTN_TC", "1") == "1"
USE_TC_BWD = os.environ.get("ARTB_ATTN_TC_BWD", "1") == "1"
_bound: dict[str, object] = {}


def _f(name: str):
    fn = _bound.get(name)
    if fn is None:
        fn = getattr(_lib.kernels(), name)
        fn.argtypes = _sigs[name]
        fn.restype = ci
        _bound[name] = fn
    return fn


def tile_states(gid: torch.Tensor, pid: torch.Tensor, S: int) -> torch.Tensor:
    """uint8 [rows, S/64, S/64]: 0 empty, 1 partially masked, 2 fully allowed."""
    M = gid.numel()
    rows, nb = M // S, S // 64
    state = torch.empty((rows, nb, nb), dtype=torch.uint8, device=gid.device)
    _lib.check_rc(_f("artb_attn_tile_states")(_lib.ptr(gid), _lib.ptr(pid), _lib.ptr(state), rows, S,
                                              _lib.stream_ptr()), "attn_tile_states")
    return state


def forward(qkv: torch.Tensor, Hq: int, Hkv: int, hd: int, plan) -> tuple[torch.Tensor, tuple]:
    M = qkv.shape[0]
    S = plan.S
    out = torch.empty((M, Hq * hd), dtype=qkv.dtype, device=qkv.device)
    lse2 = torch.empty((Hq, M), dtype=torch.float32, device=qkv.device)
    if USE_TC and hd == 128 and S % 128 == 0 and M % 8 == 0:
        vt = torch.empty((Hkv * hd, M), dtype=qkv.dtype, device=qkv.device)
        _lib.check_rc(_f("artb_attn_tc_fwd")(_lib.ptr(qkv), qkv.stride(0), _lib.ptr(plan.gid), _lib.ptr(plan.pid),
                                             _lib.ptr(plan.state), _lib.ptr(vt), _lib.ptr(out), out.stride(0),
                                             _lib.ptr(lse2), M // S, S, Hq, Hkv,
                                             _lib.ptr(_lib.status_word(qkv.device)), _lib.stream_ptr()), "attn_tc_fwd")
        return out, (qkv, out, lse2, Hq, Hkv, hd)
    _lib.check_rc(_f("artb_attn_tree_fwd")(_lib.ptr(qkv), qkv.stride(0), _lib.ptr(plan.gid), _lib.ptr(plan.pid),
                                           _lib.ptr(plan.state), _lib.ptr(out), out.stride(0), _lib.ptr(lse2),
                                           M // S, S, Hq, Hkv, hd, _lib.stream_ptr()), "attn_tree_fwd")
    return out, (qkv, out, lse2, Hq, Hkv, hd)


def backward(dout: torch.Tensor, saved: tuple, plan) -> torch.Tensor:
    qkv, out, lse2, Hq, Hkv, hd = saved
    M, S = qkv.shape[0], plan.S
    dqkv = torch.empty_like(qkv)
    dbuf = torch.empty((Hq, M), dtype=torch.float32, device=qkv.device)
    if USE_TC_BWD and hd == 128 and S % 128 == 0 and M % 8 == 0:
        qt = torch.empty((Hq * hd, M), dtype=qkv.dtype, device=qkv.device)
        dot = torch.empty((Hq * hd, M), dtype=qkv.dtype, device=qkv.device)
        kt = torch.empty((Hkv * hd, M), dtype=qkv.dtype, device=qkv.device)
        partial = torch.empty((2, M, 2 * Hkv * hd), dtype=torch.float32, device=qkv.device) if Hq // Hkv >= 4 else None
        _lib.check_rc(_f("artb_attn_tc_bwd")(_lib.ptr(qkv), qkv.stride(0), _lib.ptr(out), _lib.ptr(dout), out.stride(0),
                                             _lib.ptr(plan.gid), _lib.ptr(plan.pid), _lib.ptr(plan.state),
                                             _lib.ptr(lse2), _lib.ptr(dbuf), _lib.ptr(qt), _lib.ptr(dot), _lib.ptr(kt),
                                             _lib.ptr(dqkv), _lib.ptr(partial), M // S, S, Hq, Hkv,
                                             _lib.ptr(_lib.status_word(qkv.device)), _lib.stream_ptr()), "attn_tc_bwd")
        return dqkv
    dq_acc = torch.empty((M, Hq * hd), dtype=torch.float32, device=qkv.device)
    _lib.check_rc(_f("artb_attn_tree_bwd")(_lib.ptr(qkv), qkv.stride(0), _lib.ptr(out), _lib.ptr(dout), out.stride(0),
                                           _lib.ptr(plan.gid), _lib.ptr(plan.pid), _lib.ptr(plan.state),
                                           _lib.ptr(lse2), _lib.ptr(dbuf), _lib.ptr(dq_acc), _lib.ptr(dqkv),
                                           M // S, S, Hq, Hkv, hd, _lib.stream_ptr()), "attn_tree_bwd")
    return dqkv
