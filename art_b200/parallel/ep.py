"""Expert parallelism: all-to-all dispatch / combine of MoE token rows over NVLink peer memory.

``ExpertParallel`` owns a symmetric buffer (count table, two receive staging buffers, two return
staging buffers, flags) and drives the kernels of ``csrc/comm/moe_dispatch.cu`` and
``moe_combine.cu``:

    plan  = ops.moe.route(logits, k, norm)          # local routing over ALL experts
    rplan = ep.exchange(plan)                        # counts all-gather -> every offset of the call
    xp    = ep.dispatch(h, plan, rplan)              # rows of my experts, expert-sorted, 128-padded
    ...   grouped GEMMs over rplan (E / world local experts) ...
    yr    = ep.combine_return(yp, plan, rplan)       # expert outputs back in my own sorted order
    out   = ops.moe.combine(yr, plan, ...)           # weighted sum over each token's k experts

The backward pass dispatches ``w * dY`` and returns ``dX`` through the same calls with the saved
``rplan``.  Capacity: the receive buffer holds ``capacity_factor * M * k`` rows (plus padding).  Rows
routed to an owner beyond that are dropped by their senders: they contribute zero to the layer (and
receive a zero gradient), every owner-side offset is clipped to the buffer, and ``dropped_rows()``
counts them.  With ``drop_overflow=False`` (default) such a call also raises ``KernelStatusError``
(overflow) at the next status check; ``True`` is capacity-factor training as in GShard-style MoE.

The reference has no expert parallelism (dense models only).  ``reference_dispatch`` is the
``all_to_all_single`` restatement used by the tests.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops.moe import RoutePlan
from .symm_mem import SymmetricBuffer

_configured = False


def _k():
    global _configured
    lib = _lib.kernels()
    if not _configured:
        vp, ci, cl, cu = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_uint
        lib.artb_ep_exchange.argtypes = [vp, cl, cl, ci, vp, cu, ci, vp, ci, vp, vp]
        lib.artb_ep_dispatch.argtypes = [vp, cl, cl, cl, ci, vp, ci, ci, vp, vp, ci, vp, vp, ci, vp, ci, vp, cu, ci,
                                         ci, vp, vp]
        lib.artb_ep_recv.argtypes = [vp, cl, cl, cl, ci, ci, vp, vp, ci, ci, cu, ci, vp, vp, vp]
        lib.artb_ep_return.argtypes = [vp, cl, cl, cl, ci, vp, ci, ci, vp, ci, ci, cu, ci, vp, vp, vp]
        lib.artb_ep_ret_finish.argtypes = [vp, cl, cl, cl, ci, ci, vp, vp, vp, vp, ci, vp, ci, ci, cu, ci, vp, vp, vp]
        for f in (lib.artb_ep_exchange, lib.artb_ep_dispatch, lib.artb_ep_recv, lib.artb_ep_return,
                  lib.artb_ep_ret_finish):
            f.restype = ci
        _configured = True
    return lib


def _align(x: int, a: int = 256) -> int:
    return (x + a - 1) // a * a


@dataclass
class RecvPlan:
    """Layout of the rows this rank receives for its local experts (duck-types ``RoutePlan`` for the
    grouped GEMM / grouped wgrad: ``E`` is the number of LOCAL experts)."""
    E: int
    cap_tiles: int
    cnt_all: torch.Tensor
    send_off: torch.Tensor
    seg_off: torch.Tensor
    tile_expert: torch.Tensor
    src_start: torch.Tensor
    src_seg_off: torch.Tensor
    real_rows: torch.Tensor
    ptrs: object = None       # ctypes array of the seven device pointers

    @property
    def cap_rows(self) -> int:
        return self.cap_tiles * 128

    @property
    def total_rows(self) -> torch.Tensor:
        return self.seg_off[self.E:self.E + 1]


class ExpertParallel:
    def __init__(self, device, group, max_tokens: int, k: int, num_experts: int, d_model: int,
                 capacity_factor: float | None = 2.0, wait_ms: int = 4000, drop_overflow: bool = False):
        """``capacity_factor``: rows an owner can receive per step, as a multiple of the rows one rank sends
        (``max_tokens * k``).  ``None`` sizes the buffers for the worst case, every rank sending everything to one
        owner (= the group size): no row can ever be dropped, at ``world / 2`` times the memory of the default."""
        self.device = torch.device(device)
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if num_experts % self.world or self.world > 8:
            raise ValueError("experts must divide evenly over at most 8 ranks")
        self.E, self.El, self.k, self.D, self.wait_ms = num_experts, num_experts // self.world, k, d_model, wait_ms
        # rows routed to an owner beyond its receive capacity are dropped (they contribute zero to the layer).  With
        # drop_overflow=False that is reported as an error at the next status check; True = capacity-factor training.
        self.drop_overflow = drop_overflow
        self.cap_src_tiles = (max_tokens * k + num_experts * 127 + 127) // 128
        self.dropless = capacity_factor is None or capacity_factor >= self.world
        recv_rows = int((self.world if capacity_factor is None else capacity_factor) * max_tokens * k) + self.El * 127
        self.cap_recv_tiles = (recv_rows + 127) // 128
        P, E = self.world, self.E
        off = 0
        self.off_cnt = []
        for _ in range(2):
            self.off_cnt.append(off)
            off = _align(off + P * E * 4)
        self.off_cnt_flag = off
        off = _align(off + 64)
        self.off_recv = []
        for _ in range(2):
            self.off_recv.append(off)
            off = _align(off + self.cap_recv_tiles * 128 * d_model * 2)
        self.off_dflag = off
        off = _align(off + self.El * P * 4)
        self.off_ddone = off
        off = _align(off + 64)
        self.off_ret = []
        for _ in range(2):
            self.off_ret.append(off)
            off = _align(off + self.cap_src_tiles * 128 * d_model * 2)
        self.off_rflag = off
        off = _align(off + 64)
        self.off_rdone = off
        off = _align(off + 64)
        self.buf = SymmetricBuffer(off, self.device, group)
        self.done_cnt = torch.zeros(E, dtype=torch.int32, device=self.device)
        self.counters = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.x_epoch = self.d_epoch = self.r_epoch = 0

    @property
    def cap_recv_rows(self) -> int:
        return self.cap_recv_tiles * 128

    def _status(self):
        return _lib.ptr(_lib.status_word(self.device))

    # ------------------------------------------------------------------------------------------
    def exchange(self, plan: RoutePlan) -> RecvPlan:
        """All-gather the per-expert counts and derive the layout of this call on every rank."""
        assert plan.E == self.E and plan.cap_tiles <= self.cap_src_tiles
        dev, P, E, El = self.device, self.world, self.E, self.El
        i32 = dict(dtype=torch.int32, device=dev)
        rp = RecvPlan(El, self.cap_recv_tiles, torch.empty(P * E, **i32), torch.empty(E, **i32),
                      torch.empty(El + 1, **i32), torch.empty(self.cap_recv_tiles, **i32), torch.empty(El * P, **i32),
                      torch.empty(P * El, **i32), torch.empty(El, **i32))
        rp.ptrs = (ctypes.c_void_p * 7)(*(t.data_ptr() for t in (rp.cnt_all, rp.send_off, rp.seg_off, rp.tile_expert,
                                                                   rp.src_start, rp.src_seg_off, rp.real_rows)))
        self.x_epoch += 1
        rc = _k().artb_ep_exchange(self.buf._h, self.off_cnt[self.x_epoch & 1], self.off_cnt_flag, E,
                                   _lib.ptr(plan.counts), self.x_epoch, self.wait_ms, rp.ptrs, self.cap_recv_tiles,
                                   self._status(), _lib.stream_ptr())
        _lib.check_rc(rc, "ep_exchange")
        return rp

    def dispatch(self, x: torch.Tensor, plan: RoutePlan, rp: RecvPlan, weighted: bool = False) -> torch.Tensor:
        """Rows ``x[token]`` (times the routing weight if ``weighted``) to their experts' owners.

        Returns this rank's received rows ``[cap_recv_rows, D]`` in local-expert order (private memory)."""
        D = x.shape[1]
        assert D == self.D
        self.d_epoch += 1
        par = self.d_epoch & 1
        st = _lib.stream_ptr()
        rc = _k().artb_ep_dispatch(self.buf._h, self.off_recv[par], self.off_dflag, self.off_ddone, self.E, _lib.ptr(x),
                                   x.stride(0), D, _lib.ptr(plan.row_token), _lib.ptr(plan.row_w), int(weighted),
                                   _lib.ptr(plan.seg_off), _lib.ptr(plan.tile_expert), plan.cap_rows, rp.ptrs,
                                   self.cap_recv_rows, _lib.ptr(self.done_cnt), self.d_epoch, self.wait_ms,
                                   int(self.drop_overflow), self._status(), st)
        _lib.check_rc(rc, "ep_dispatch")
        out = torch.empty((self.cap_recv_rows, D), dtype=torch.bfloat16, device=self.device)
        rc = _k().artb_ep_recv(self.buf._h, self.off_recv[par], self.off_dflag, self.off_ddone, self.E, D, rp.ptrs,
                               _lib.ptr(out), out.stride(0), self.cap_recv_rows, self.d_epoch, self.wait_ms,
                               self._status(), self.counters[0:1].data_ptr(), st)
        _lib.check_rc(rc, "ep_recv")
        return out

    def combine_return(self, yp: torch.Tensor, plan: RoutePlan, rp: RecvPlan) -> torch.Tensor:
        """Expert-ordered rows back to their sources; returns ``[plan.cap_rows, D]`` in this rank's sorted order."""
        D = yp.shape[1]
        assert D == self.D and yp.shape[0] == self.cap_recv_rows
        self.r_epoch += 1
        par = self.r_epoch & 1
        st = _lib.stream_ptr()
        rc = _k().artb_ep_return(self.buf._h, self.off_ret[par], self.off_rflag, self.off_rdone, self.E, _lib.ptr(yp),
                                 yp.stride(0), D, rp.ptrs, self.cap_recv_rows, self.cap_src_tiles * 128, self.r_epoch,
                                 self.wait_ms, self._status(), self.counters[1:2].data_ptr(), st)
        _lib.check_rc(rc, "ep_return")
        out = torch.empty((plan.cap_rows, D), dtype=torch.bfloat16, device=self.device)
        rc = _k().artb_ep_ret_finish(self.buf._h, self.off_ret[par], self.off_rflag, self.off_rdone, self.E, D,
                                     _lib.ptr(plan.row_token), _lib.ptr(plan.seg_off), _lib.ptr(plan.tile_expert),
                                     _lib.ptr(rp.send_off), self.cap_recv_rows, _lib.ptr(out), out.stride(0), plan.cap_rows,
                                     self.r_epoch, self.wait_ms, self._status(), self.counters[2:3].data_ptr(), st)
        _lib.check_rc(rc, "ep_ret_finish")
        return out

    def dropped_rows(self, reset: bool = True) -> int:
        """Rows dropped for lack of capacity since the last call (one device-to-host read)."""
        w = _lib.status_word(self.device)
        n = int(w[1].item())
        if reset:
            w[1] = 0
        return n

    def close(self) -> None:
        self.buf.close()


def reference_exchange_layout(cnt_all: torch.Tensor, rank: int, cap_tiles: int) -> dict[str, torch.Tensor]:
    """Plain-Python restatement of the offsets the exchange kernel derives on ``rank`` from the gathered counts
    ``cnt_all`` [P, E] (tokens of source s routed to expert e), for a receive buffer of ``cap_tiles`` 128-row tiles.

    * ``send_off[e]``: row in the owner's receive buffer where this rank's rows for expert e start (sources are laid
      out in rank order inside an expert's segment, segments are padded to 128 rows);
    * owner side, clipped to the capacity: ``seg_off`` [El + 1], ``real_rows`` [El], ``tile_expert`` [cap_tiles]
      (-1 beyond the last segment), ``src_start`` [El, P] (first row of source s inside segment j) and
      ``src_seg_off`` [P, El] (where expert j's segment starts in source s's own sorted order).
    A sender drops row i of expert e when ``send_off[e] + i >= cap_tiles * 128``; the clipped ``real_rows`` are exactly
    the rows that were not dropped."""
    cnt = cnt_all.to(torch.int64).cpu()
    P, E = cnt.shape
    El = E // P
    cap = cap_tiles * 128
    pad = lambda n: (int(n) + 127) // 128 * 128  # noqa: E731
    send_off = torch.zeros(E, dtype=torch.int64)
    for e in range(E):
        owner, j = divmod(e, El)
        seg = sum(pad(cnt[:, owner * El + j2].sum()) for j2 in range(j))
        send_off[e] = seg + int(cnt[:rank, e].sum())
    seg_off = torch.zeros(El + 1, dtype=torch.int64)
    real = torch.zeros(El, dtype=torch.int64)
    src_start = torch.zeros(El, P, dtype=torch.int64)
    src_seg_off = torch.zeros(P, El, dtype=torch.int64)
    seg = 0
    for j in range(El):
        e = rank * El + j
        tot = int(cnt[:, e].sum())
        seg_c = min(seg, cap)
        seg_off[j] = seg_c
        real[j] = min(tot, cap - seg_c)
        run = 0
        for s_ in range(P):
            src_start[j, s_] = run
            run += int(cnt[s_, e])
            src_seg_off[s_, j] = sum(pad(cnt[s_, e2]) for e2 in range(e))
        seg += pad(tot)
    seg_off[El] = max(min(seg, cap), int(seg_off[El - 1]))
    tile_expert = torch.full((cap_tiles,), -1, dtype=torch.int64)
    for t in range(cap_tiles):
        row = t * 128
        if row < int(seg_off[El]):
            tile_expert[t] = max(j for j in range(El) if int(seg_off[j]) <= row)
    return {"send_off": send_off, "seg_off": seg_off, "real_rows": real, "tile_expert": tile_expert,
            "src_start": src_start, "src_seg_off": src_seg_off}


def reference_dispatch(x: torch.Tensor, topi: torch.Tensor, num_experts: int, group=None):
    """NCCL restatement: returns (rows for my experts sorted by (expert, source, token order), expert id per row)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    El = num_experts // world
    M, k = topi.shape
    tok = torch.arange(M, device=x.device).repeat_interleave(k)
    e = topi.reshape(-1).long()
    order = torch.argsort(e, stable=True)
    e_s, tok_s = e[order], tok[order]
    send_counts = torch.bincount(e_s // El, minlength=world)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    sc, rc = send_counts.tolist(), recv_counts.tolist()
    rows = torch.empty((sum(rc), x.shape[1]), dtype=x.dtype, device=x.device)
    dist.all_to_all_single(rows, x[tok_s].contiguous(), rc, sc, group=group)
    eid = torch.empty(sum(rc), dtype=torch.long, device=x.device)
    dist.all_to_all_single(eid, e_s.contiguous(), rc, sc, group=group)
    return rows, eid - rank * El
