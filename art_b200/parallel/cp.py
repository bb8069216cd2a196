"""Context parallelism for long packed rows: zig-zag token sharding + K/V exchange over NVLink.

A packed row of ``S`` tokens is cut into ``2P`` chunks and rank ``r`` owns chunks ``r`` and
``2P-1-r`` (balanced causal work).  Every token-wise layer runs on the ``S/P`` local tokens; for
attention each rank holds a full-length ``q|k|v`` buffer in symmetric memory whose K/V columns the
peers fill by pushing their rows (``csrc/comm/ring_attn.cu``), then runs the single-GPU tree-mask
kernels with the tile states of non-local query blocks cleared.  The backward sums the partial
``dK|dV`` of all ranks at the owner of each token.

Buffers are indexed by (layer, call parity): a peer cannot be two calls ahead on the same layer
because every call consumes that peer's data, and the slot a forward pass saved for its backward is
only overwritten by the forward of the next micro-batch, which starts after the peers have received
this rank's ``dK|dV`` for that layer, i.e. after this rank's last read of the slot.

The reference has no context parallelism (``src/art/local/train.py:177-215`` builds one dense
``[B,S,S]`` bias on one GPU).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import _lib, attn_native
from ..ops.attention import AttnCtx, AttnPlan
from .symm_mem import SymmetricBuffer

_configured = False


def _k():
    global _configured
    lib = _lib.kernels()
    if not _configured:
        vp, ci, cl, cu = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_uint
        lib.artb_cp_kv_exchange.argtypes = [vp, cl, cl, vp, ci, ci, vp, ci, cu, ci, vp, vp, vp]
        lib.artb_cp_kv_exchange.restype = ci
        lib.artb_cp_dkv_reduce.argtypes = [vp, cl, cl, vp, ci, ci, vp, vp, vp, cl, ci, vp, ci, cu, ci, vp, vp, vp]
        lib.artb_cp_dkv_reduce.restype = ci
        _configured = True
    return lib


def zigzag_owner(S: int, world: int) -> torch.Tensor:
    """int32 [S]: owning rank of every position of a packed row."""
    if S % (2 * world * 64):
        raise ValueError("row length must be a multiple of 128 * world (64-token tiles, two chunks per rank)")
    chunk = S // (2 * world)
    c = torch.arange(S) // chunk
    return torch.where(c < world, c, 2 * world - 1 - c).to(torch.int32)


def _align(x: int, a: int = 256) -> int:
    return (x + a - 1) // a * a


class ContextParallel:
    def __init__(self, device, group, rows: int, S: int, Hq: int, Hkv: int, hd: int, num_layers: int,
                 wait_ms: int = 4000):
        self.device = torch.device(device)
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.rows, self.S, self.Hq, self.Hkv, self.hd, self.L = rows, S, Hq, Hkv, hd, num_layers
        self.wait_ms = wait_ms
        P = self.world
        own = zigzag_owner(S, P)
        self.S_loc = S // P
        owner_full = own.repeat(rows)                                        # [rows*S]
        g = torch.arange(rows * S)
        mine = g[owner_full == self.rank]
        self.local_to_global = mine.to(torch.int32).to(self.device)          # [rows*S_loc], row-major
        lidx = torch.zeros(rows * S, dtype=torch.int32)
        for r in range(P):
            sel = owner_full == r
            lidx[sel] = torch.arange(int(sel.sum()), dtype=torch.int32)
        self.owner_of = owner_full.to(self.device)
        self.local_index_of = lidx.to(self.device)
        self.n_local, self.n_global = rows * self.S_loc, rows * S
        self.ld = (Hq + 2 * Hkv) * hd
        self.kv0 = Hq * hd
        nb = S // 64
        qb_owner = own.view(nb, 64)[:, 0]
        self.nonlocal_qb = (qb_owner != self.rank).nonzero().squeeze(1).to(self.device)
        off = 0
        self.off_full = []
        for _ in range(2 * num_layers):
            self.off_full.append(off)
            off = _align(off + self.n_global * self.ld * 2)
        self.off_kv_flag = off
        off = _align(off + 64)
        self.off_stage = []
        kvw = 2 * Hkv * hd
        for _ in range(2):
            self.off_stage.append(off)
            off = _align(off + P * self.n_local * kvw * 2)
        self.off_dkv_flag = off
        off = _align(off + 64)
        self.buf = SymmetricBuffer(off, self.device, group)
        self._bytes = self.buf.view(torch.uint8)
        self.counters = torch.zeros(2, dtype=torch.int32, device=self.device)
        self.calls = [0] * num_layers
        self.fwd_epoch = 0
        self.bwd_epoch = 0

    # ---------------------------------------------------------------------------------------------
    def shard(self, t: torch.Tensor) -> torch.Tensor:
        """Rows of a ``[rows*S, ...]`` tensor that this rank owns, in local order."""
        return t[self.local_to_global.long()]

    def make_plan(self, gid_full: torch.Tensor, pid_full: torch.Tensor) -> AttnPlan:
        """Tile states of the full rows with the query blocks of other ranks cleared."""
        plan = AttnPlan("native", gid_full, pid_full, self.S)
        state = attn_native.tile_states(gid_full, pid_full, self.S)
        state[:, self.nonlocal_qb, :] = 0
        plan.state = state
        return plan

    def _full_view(self, layer: int, parity: int) -> torch.Tensor:
        off = self.off_full[2 * layer + parity]
        n = self.n_global * self.ld * 2
        return self._bytes[off:off + n].view(torch.bfloat16).view(self.n_global, self.ld)

    def forward(self, layer: int, qkv_local: torch.Tensor, plan: AttnPlan) -> tuple[torch.Tensor, AttnCtx]:
        """``qkv_local`` [n_local, ld] post-RoPE -> local attention output [n_local, Hq*hd]."""
        assert qkv_local.shape == (self.n_local, self.ld) and qkv_local.stride(1) == 1
        self.calls[layer] += 1
        par = self.calls[layer] & 1
        self.fwd_epoch += 1
        rc = _k().artb_cp_kv_exchange(self.buf._h, self.off_full[2 * layer + par], self.off_kv_flag,
                                      _lib.ptr(qkv_local), qkv_local.stride(0), self.kv0,
                                      _lib.ptr(self.local_to_global), self.n_local, self.fwd_epoch, self.wait_ms,
                                      self.counters[0:1].data_ptr(), _lib.ptr(_lib.status_word(self.device)),
                                      _lib.stream_ptr())
        _lib.check_rc(rc, "cp_kv_exchange")
        full = self._full_view(layer, par)
        if qkv_local.stride(0) != self.ld:
            raise ValueError("qkv_local must be dense")
        o_full, saved = attn_native.forward(full, self.Hq, self.Hkv, self.hd, plan)
        o_local = o_full[self.local_to_global.long()]
        return o_local, AttnCtx(plan, (saved, o_full))

    def backward(self, do_local: torch.Tensor, ctx: AttnCtx) -> torch.Tensor:
        saved, o_full = ctx.saved
        do_full = torch.zeros_like(o_full)
        do_full[self.local_to_global.long()] = do_local
        dqkv_full = attn_native.backward(do_full, saved, ctx.plan)
        self.bwd_epoch += 1
        par = self.bwd_epoch & 1
        out = torch.empty((self.n_local, self.ld), dtype=torch.bfloat16, device=self.device)
        rc = _k().artb_cp_dkv_reduce(self.buf._h, self.off_stage[par], self.off_dkv_flag, _lib.ptr(dqkv_full),
                                     dqkv_full.stride(0), self.kv0, _lib.ptr(self.owner_of),
                                     _lib.ptr(self.local_index_of), _lib.ptr(self.local_to_global), self.n_global,
                                     self.n_local, _lib.ptr(out), out.stride(0), self.bwd_epoch, self.wait_ms,
                                     self.counters[1:2].data_ptr(), _lib.ptr(_lib.status_word(self.device)),
                                     _lib.stream_ptr())
        _lib.check_rc(rc, "cp_dkv_reduce")
        return out

    def close(self) -> None:
        self._bytes = None
        self.buf.close()
