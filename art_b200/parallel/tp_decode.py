"""Decode-side tensor parallelism pieces: row-parallel small-M GEMM with the all-reduce fused into its
finalize pass, and the device-memory LoRA hand-off between a trainer rank and engine ranks
(``csrc/comm/gemm_ar_decode.cu``).

The reference reaches a tensor-parallel decode only through the inference library's ``tensor_parallel_size``
(``src/art/dev/engine.py:27``) and hands adapters over through files (``src/art/local/service.py:150-174``).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops.gemm import gemm_splitk_, plan_small_m
from .symm_mem import SymmetricBuffer

_configured = False


def _k():
    global _configured
    lib = _lib.kernels()
    if not _configured:
        vp, ci, cl, cu = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_uint
        lib.artb_splitk_finalize_allreduce.argtypes = [vp, cl, cl, cl, vp, ci, ci, vp, vp, ci, ci, vp, ci, cu, ci, vp, vp]
        lib.artb_lora_push.argtypes = [vp, cl, cl, vp, cl, cu, vp, vp]
        lib.artb_lora_wait.argtypes = [vp, cl, ci, cu, ci, vp, vp]
        for f in (lib.artb_splitk_finalize_allreduce, lib.artb_lora_push, lib.artb_lora_wait):
            f.restype = ci
        _configured = True
    return lib


def _align(x: int, a: int = 256) -> int:
    return (x + a - 1) // a * a


class DecodeAllReduce:
    """``out = sum_p x_p @ w_p.T (+ bias + residual)`` on every rank, for M of a few hundred rows."""

    def __init__(self, device, group, max_rows: int, max_cols: int, wait_ms: int = 4000):
        self.device, self.group = torch.device(device), group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.stride = _align(max_rows * max_cols, 1024)
        n_slices = self.stride // 1024
        self.off_stage = [0, _align(self.world * self.stride * 4)]
        self.off_flag = 2 * _align(self.world * self.stride * 4)
        self.buf = SymmetricBuffer(self.off_flag + _align(self.world * n_slices * 4), self.device, group)
        self.ws = torch.zeros(self.stride, dtype=torch.float32, device=self.device)
        self.epoch, self.wait_ms = 0, wait_ms

    def gemm_allreduce(self, x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
                       residual: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
        M, K = x.shape
        N = w.shape[0]
        if M * N > self.stride or N % 8:
            raise ValueError("shape outside the workspace")
        ws = self.ws[:M * N].view(M, N)
        bn, splits = plan_small_m(M, N, K)
        gemm_splitk_(ws, x, w, bn, splits)
        if out is None:
            out = torch.empty((M, N), dtype=torch.bfloat16, device=self.device)
        self.epoch += 1
        rc = _k().artb_splitk_finalize_allreduce(
            self.buf._h, self.off_stage[self.epoch & 1], self.off_flag, self.stride, _lib.ptr(ws), M, N, _lib.ptr(bias),
            _lib.ptr(residual), residual.stride(0) if residual is not None else 0, 0, _lib.ptr(out), out.stride(0),
            self.epoch, self.wait_ms, _lib.ptr(_lib.status_word(self.device)), _lib.stream_ptr())
        _lib.check_rc(rc, "splitk_finalize_allreduce")
        return out

    def close(self) -> None:
        self.buf.close()


class LoraHandoff:
    """Flat fp32 LoRA buffer pushed from one rank into the others' device memory (no file, no host copy)."""

    def __init__(self, device, group, numel: int, wait_ms: int = 4000):
        self.device, self.group = torch.device(device), group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.n = (numel + 3) // 4 * 4
        self.off_flag = _align(self.n * 4)
        self.buf = SymmetricBuffer(self.off_flag + 256, self.device, group)
        self.counter = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.epoch, self.wait_ms = 0, wait_ms

    def push(self, flat: torch.Tensor) -> None:
        assert flat.dtype == torch.float32 and flat.is_contiguous() and flat.numel() <= self.n and flat.numel() % 4 == 0
        self.epoch += 1
        _lib.check_rc(_k().artb_lora_push(self.buf._h, 0, self.off_flag, _lib.ptr(flat), flat.numel(), self.epoch,
                                          self.counter.data_ptr(), _lib.stream_ptr()), "lora_push")

    def receive(self, src: int, numel: int) -> torch.Tensor:
        """Wait (on the stream) for the next push of ``src`` and return a view of the received parameters."""
        self.epoch += 1
        _lib.check_rc(_k().artb_lora_wait(self.buf._h, self.off_flag, src, self.epoch, self.wait_ms,
                                          _lib.ptr(_lib.status_word(self.device)), _lib.stream_ptr()), "lora_wait")
        return self.buf.view(torch.float32, numel)

    def close(self) -> None:
        self.buf.close()
