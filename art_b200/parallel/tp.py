"""Tensor parallelism with token-sharded activations: fused all-gather->GEMM and GEMM->reduce-scatter.

A ``TPContext`` owns one symmetric (peer-mapped) buffer per process and carves it into the
regions the two kernels of ``csrc/comm`` need:

* all-gather side: two copies (epoch parity) of the gathered activation matrix ``X`` and of the
  gathered LoRA low-rank activations ``T``, arrival flags, "done" words;
* reduce-scatter side: two copies of the bf16 staging area that peers push partial tiles into,
  per-tile flags, "done" words.

Column-parallel linears (q/k/v, gate/up) call :meth:`ag_gemm` after writing their token shard
into :meth:`ag_input`; row-parallel linears (o, down) call :meth:`gemm_rs`.  The same two calls
serve the backward data-gradients with the roles swapped.

The reference has no tensor parallelism of its own; ``tensor_parallel_size`` is forwarded to the
inference library (``src/art/dev/engine.py:27``).  ``unfused_ag_gemm`` / ``unfused_gemm_rs`` are
the NCCL + matmul baselines the fused kernels are measured against.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops.gemm import EPI_BF16, EPI_F32, EPI_SWIGLU, EPI_SWIGLU_BWD
from .symm_mem import SymmetricBuffer

_configured = False
PUSH_ROWS = 32


def _k():
    global _configured
    lib = _lib.kernels()
    if not _configured:
        vp, ci, cl, cu = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_uint
        lib.artb_tp_ag_gemm.argtypes = [vp, cl, cl, ci, cl, cl, vp, ci, vp, ci, vp, ci, vp, ci, vp, ci, ci, ci, ci,
                                        cu, ci, vp, vp, ci, vp]
        lib.artb_tp_ag_gemm.restype = ci
        lib.artb_tp_gemm_rs.argtypes = [vp, cl, cl, cl, ci, vp, ci, vp, ci, vp, ci, vp, ci, ci, vp, ci, vp, ci, ci,
                                        ci, ci, cu, ci, vp, vp, ci, vp]
        lib.artb_tp_gemm_rs.restype = ci
        _configured = True
    return lib


def _align(x: int, a: int = 256) -> int:
    return (x + a - 1) // a * a


class TPContext:
    """Symmetric workspace + call counters of one tensor-parallel group (one per process)."""

    def __init__(self, device, group, m_seg: int, k_max: int, n_max: int, kt: int = 64, wait_ms: int = 4000):
        if m_seg % 128:
            raise ValueError("tokens per rank must be a multiple of 128")
        self.device = torch.device(device)
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if self.world > 8:
            raise ValueError("tensor-parallel groups of at most 8 ranks")
        self.m_seg, self.k_max, self.n_max, self.kt, self.wait_ms = m_seg, k_max, n_max, kt, wait_ms
        M = self.world * m_seg
        off = 0
        self.off_x = []
        self.off_t = []
        for _ in range(2):
            self.off_x.append(off)
            off = _align(off + M * k_max * 2)
            self.off_t.append(off)
            off = _align(off + M * kt * 2)
        self.off_ag_flag = off
        off = _align(off + self.world * (m_seg // PUSH_ROWS) * 4)
        self.off_ag_done = off
        off = _align(off + 64)
        self.tile_cap = (m_seg // 128) * ((n_max + 127) // 128)
        self.off_stage = []
        for _ in range(2):
            self.off_stage.append(off)
            off = _align(off + max(self.world - 1, 1) * m_seg * n_max * 2)
        self.off_rs_flag = off
        off = _align(off + max(self.world - 1, 1) * self.tile_cap * 32)    # 8 epilogue warps per tile, one flag each
        self.off_rs_done = off
        off = _align(off + 64)
        self.buf = SymmetricBuffer(off, self.device, group)
        self._bytes = self.buf.view(torch.uint8)
        self.counters = torch.zeros(2, dtype=torch.int32, device=self.device)
        self.ag_epoch = 0
        self.rs_epoch = 0

    # ------------------------------------------------------------------ all-gather -> GEMM
    def _region(self, off: int, rows: int, cols: int, dtype=torch.bfloat16) -> torch.Tensor:
        nbytes = rows * cols * torch.empty((), dtype=dtype).element_size()
        return self._bytes[off:off + nbytes].view(dtype).view(rows, cols)

    def ag_input(self, K: int) -> torch.Tensor:
        """[m_seg, K] view the caller fills with its token shard before the next :meth:`ag_gemm`."""
        if K > self.k_max:
            raise ValueError("K exceeds the workspace")
        par = (self.ag_epoch + 1) & 1
        full = self._region(self.off_x[par], self.world * self.m_seg, K)
        return full[self.rank * self.m_seg:(self.rank + 1) * self.m_seg]

    def ag_t_input(self) -> torch.Tensor:
        """[m_seg, kt] view for the shard of the LoRA low-rank activations gathered with X."""
        par = (self.ag_epoch + 1) & 1
        full = self._region(self.off_t[par], self.world * self.m_seg, self.kt)
        return full[self.rank * self.m_seg:(self.rank + 1) * self.m_seg]

    def ag_gemm(self, K: int, b: torch.Tensor, b2: torch.Tensor | None = None, out: torch.Tensor | None = None,
                swiglu_out: torch.Tensor | None = None, bias: torch.Tensor | None = None,
                out_dtype: torch.dtype = torch.bfloat16, max_ctas: int = 0,
                swiglu_bwd_gu: torch.Tensor | None = None):
        """``out[M, N] = gather(X) @ b.T (+ gather(T) @ b2.T)``; returns ``(out, x_full, t_full)``.

        ``x_full`` / ``t_full`` are views of the gathered operands; they stay valid until the
        second-next call of this method.  ``swiglu_bwd_gu`` ([M, 2N], the forward's interleaved gate|up
        pre-activations): the product is d(silu(gate) * up) and ``out`` ([M, 2N]) receives d(gate|up).
        """
        self.ag_epoch += 1
        par = self.ag_epoch & 1
        N = b.shape[0]
        M = self.world * self.m_seg
        if b.shape[1] != K or b.stride(1) != 1:
            raise ValueError("weight shard must be [N, K] with unit inner stride")
        epi = EPI_SWIGLU if swiglu_out is not None else (EPI_F32 if out_dtype == torch.float32 else EPI_BF16)
        if swiglu_bwd_gu is not None:
            if tuple(swiglu_bwd_gu.shape) != (M, 2 * N) or N % 32 or swiglu_bwd_gu.stride(1) != 1:
                raise ValueError("swiglu_bwd_gu must be [M, 2N] with N a multiple of 32")
            epi, swiglu_out = EPI_SWIGLU_BWD, swiglu_bwd_gu      # travels in the H slot of the C entry point
            if out is None:
                out = torch.empty((M, 2 * N), dtype=torch.bfloat16, device=self.device)
        if out is None:
            out = torch.empty((M, N), dtype=torch.float32 if epi == EPI_F32 else torch.bfloat16, device=self.device)
        kt = self.kt if b2 is not None else 0
        rc = _k().artb_tp_ag_gemm(
            self.buf._h, self.off_x[par], self.off_t[par], kt, self.off_ag_flag, self.off_ag_done,
            _lib.ptr(b), b.stride(0), _lib.ptr(b2), b2.stride(0) if b2 is not None else 0,
            _lib.ptr(out), out.stride(0), _lib.ptr(swiglu_out), swiglu_out.stride(0) if swiglu_out is not None else 0,
            _lib.ptr(bias), self.m_seg, N, K, epi, self.ag_epoch, self.wait_ms,
            self.counters[0:1].data_ptr(), _lib.ptr(_lib.status_word(self.device)), max_ctas, _lib.stream_ptr())
        _lib.check_rc(rc, "tp_ag_gemm")
        x_full = self._region(self.off_x[par], M, K)
        t_full = self._region(self.off_t[par], M, self.kt) if b2 is not None else None
        return out, x_full, t_full

    # ---------------------------------------------------------------- GEMM -> reduce-scatter
    def gemm_rs(self, a: torch.Tensor, b: torch.Tensor, a2: torch.Tensor | None = None,
                b2: torch.Tensor | None = None, residual: torch.Tensor | None = None,
                out: torch.Tensor | None = None, max_ctas: int = 0) -> torch.Tensor:
        """``out[m_seg, N] = rows of this rank of sum_p (a_p @ b_p.T + a2_p @ b2.T) (+ residual)``."""
        M, K = a.shape
        N = b.shape[0]
        if M != self.world * self.m_seg or N > self.n_max:
            raise ValueError("shape outside the workspace")
        self.rs_epoch += 1
        par = self.rs_epoch & 1
        if out is None:
            out = torch.empty((self.m_seg, N), dtype=torch.bfloat16, device=self.device)
        K2 = a2.shape[1] if a2 is not None else 0
        rc = _k().artb_tp_gemm_rs(
            self.buf._h, self.off_stage[par], self.off_rs_flag, self.off_rs_done, self.tile_cap,
            _lib.ptr(a), a.stride(0), _lib.ptr(b), b.stride(0),
            _lib.ptr(a2), a2.stride(0) if a2 is not None else 0, _lib.ptr(b2), b2.stride(0) if b2 is not None else 0,
            K2, _lib.ptr(out), out.stride(0), _lib.ptr(residual), residual.stride(0) if residual is not None else 0,
            self.m_seg, N, K, self.rs_epoch, self.wait_ms, self.counters[1:2].data_ptr(),
            _lib.ptr(_lib.status_word(self.device)), max_ctas, _lib.stream_ptr())
        _lib.check_rc(rc, "tp_gemm_rs")
        return out

    def close(self) -> None:
        self._bytes = None
        self.buf.close()


# ----------------------------------------------------------------------------- unfused baselines
def unfused_ag_gemm(x_shard: torch.Tensor, b: torch.Tensor, group=None) -> torch.Tensor:
    """NCCL all_gather followed by a library matmul (the baseline the fused kernel is compared with)."""
    world = dist.get_world_size(group)
    full = torch.empty((world * x_shard.shape[0], x_shard.shape[1]), dtype=x_shard.dtype, device=x_shard.device)
    dist.all_gather_into_tensor(full, x_shard.contiguous(), group=group)
    return full @ b.t()


def unfused_gemm_rs(a: torch.Tensor, b: torch.Tensor, group=None) -> torch.Tensor:
    """Library matmul followed by an NCCL reduce_scatter along tokens."""
    world = dist.get_world_size(group)
    part = a @ b.t()
    out = torch.empty((a.shape[0] // world, b.shape[0]), dtype=part.dtype, device=part.device)
    dist.reduce_scatter_tensor(out, part, group=group)
    return out
