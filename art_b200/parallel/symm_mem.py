"""Symmetric (peer-mapped) device buffers and the collectives that run on them.

``SymmetricBuffer`` allocates the same number of bytes on every rank of a process group,
exchanges CUDA IPC handles through ``torch.distributed`` and maps every peer's allocation, so
that the kernels in ``csrc/comm`` can load from and store to remote memory over NVLink.  Buffers
come with a signal pad of epoch counters used for bounded-wait barriers between GPUs.

Nothing comparable exists in the reference (single GPU, no collectives); the closest knob is
the pass-through ``tensor_parallel_size`` (``src/art/dev/engine.py:26-27``).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import _lib

vp, ci, cl, cf, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_float, ctypes.c_size_t
_configured = False


def _k():
    global _configured
    lib = _lib.kernels()
    if not _configured:
        lib.artb_symm_create.argtypes = [ci, ci, sz]
        lib.artb_symm_create.restype = vp
        lib.artb_symm_export.argtypes = [vp, vp]
        lib.artb_symm_export.restype = ci
        lib.artb_symm_import.argtypes = [vp, ci, vp]
        lib.artb_symm_import.restype = ci
        lib.artb_symm_local_ptr.argtypes = [vp]
        lib.artb_symm_local_ptr.restype = vp
        lib.artb_symm_peer_ptr.argtypes = [vp, ci]
        lib.artb_symm_peer_ptr.restype = vp
        lib.artb_symm_destroy.argtypes = [vp]
        lib.artb_symm_reset.argtypes = [vp]
        lib.artb_lora_grad_allreduce.argtypes = [vp, cl, cf, ci, vp, vp]
        lib.artb_lora_grad_allreduce.restype = ci
        _configured = True
    return lib


class _DevicePtr:
    """Minimal ``__cuda_array_interface__`` carrier so torch can view foreign device memory."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class SymmetricBuffer:
    def __init__(self, nbytes: int, device: torch.device, group=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.device = torch.device(device)
        self.nbytes = nbytes
        with torch.cuda.device(self.device):
            self._h = _k().artb_symm_create(self.rank, self.world, nbytes)
        if not self._h:
            raise RuntimeError("symmetric allocation failed")
        handle = ctypes.create_string_buffer(64)
        _lib.check_rc(_k().artb_symm_export(self._h, handle), "symm_export")
        handles: list = [None] * self.world
        dist.all_gather_object(handles, bytes(handle.raw), group=group)
        with torch.cuda.device(self.device):
            for peer, hb in enumerate(handles):
                _lib.check_rc(_k().artb_symm_import(self._h, peer, ctypes.create_string_buffer(hb, 64)), "symm_import")
        dist.barrier(group)
        self._bytes = torch.as_tensor(_DevicePtr(_k().artb_symm_local_ptr(self._h), nbytes), device=self.device)

    def view(self, dtype: torch.dtype, numel: int | None = None) -> torch.Tensor:
        t = self._bytes.view(dtype)
        return t if numel is None else t[:numel]

    def peer_ptr(self, peer: int) -> int:
        return int(_k().artb_symm_peer_ptr(self._h, peer))

    def reset_failure(self) -> None:
        _k().artb_symm_reset(self._h)

    def close(self) -> None:
        h, self._h = self._h, None
        if h:
            self._bytes = None
            _k().artb_symm_destroy(h)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class FusedGradAllReduce:
    """Callable ``(flat_grads) -> None``: mean (or sum, ``average=False``) over ranks, in place, through the P2P kernel."""

    def __init__(self, device: torch.device, world: int, group=None, wait_ms: int = 5000, average: bool = True):
        self.device, self.world, self.group, self.wait_ms = torch.device(device), world, group, wait_ms
        self.scale = 1.0 / world if average else 1.0
        self.buf: SymmetricBuffer | None = None
        self.n = 0

    def __call__(self, flat_grads: torch.Tensor) -> None:
        n = flat_grads.numel()
        pad = (-n) % (4 * self.world)
        if self.buf is None or self.n != n + pad:
            self.n = n + pad
            self.buf = SymmetricBuffer(self.n * 4, self.device, self.group)
        sym = self.buf.view(torch.float32, self.n)
        sym[:n].copy_(flat_grads)
        if pad:
            sym[n:].zero_()
        rc = _k().artb_lora_grad_allreduce(self.buf._h, self.n, self.scale, self.wait_ms,
                                           _lib.ptr(_lib.status_word(self.device)), _lib.stream_ptr())
        _lib.check_rc(rc, "lora_grad_allreduce")
        flat_grads.copy_(sym[:n])


def fused_allreduce_sync(device: torch.device, world: int, group=None) -> FusedGradAllReduce:
    return FusedGradAllReduce(device, world, group)
