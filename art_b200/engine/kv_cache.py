"""Paged KV cache: host-side block accounting (C++ ``csrc/engine/block_manager.cpp``) and the
per-layer device tensors ``[num_blocks, block_size, Hkv, hd]``.

With ``enable_sleep_mode`` the cache can be dropped (``discard``) or copied to pinned host
memory (``offload`` / ``restore``) while the trainer owns the GPU, mirroring the two sleep
levels of the reference (``src/art/local/vllm.py:148-231``, ``state.py:146-171``).  On a
180 GB device the default is to keep it resident.
"""
from __future__ import annotations

import ctypes

import torch

from ..ops import _lib

_configured = False


def _rt():
    global _configured
    lib = _lib.runtime()
    if not _configured:
        vp, ci, u64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint64
        lib.artb_bm_create.argtypes = [ci, ci, ci]
        lib.artb_bm_create.restype = vp
        lib.artb_bm_destroy.argtypes = [vp]
        lib.artb_bm_num_free.argtypes = [vp]
        lib.artb_bm_num_free.restype = ci
        lib.artb_bm_alloc.argtypes = [vp, ci, vp]
        lib.artb_bm_alloc.restype = ci
        lib.artb_bm_free.argtypes = [vp, vp, ci]
        lib.artb_bm_match_prefix.argtypes = [vp, vp, ci, u64, vp, ci]
        lib.artb_bm_match_prefix.restype = ci
        lib.artb_bm_commit.argtypes = [vp, vp, ci, vp, ci, u64]
        lib.artb_bm_reset_cache.argtypes = [vp]
        lib.artb_bm_stats.argtypes = [vp, vp]
        _configured = True
    return lib


class BlockManager:
    """Thin wrapper over the native block manager (ref-counted blocks + prefix cache)."""

    def __init__(self, num_blocks: int, block_size: int, enable_prefix_caching: bool = True):
        self.num_blocks, self.block_size = num_blocks, block_size
        self._h = _rt().artb_bm_create(num_blocks, block_size, 1 if enable_prefix_caching else 0)
        if not self._h:
            raise ValueError("invalid block manager geometry")

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            try:
                _rt().artb_bm_destroy(h)
            except Exception:   # interpreter shutdown: the library handle may already be gone
                pass

    @property
    def num_free(self) -> int:
        return _rt().artb_bm_num_free(self._h)

    def alloc(self, n: int) -> list[int] | None:
        if n <= 0:
            return []
        buf = (ctypes.c_int * n)()
        if _rt().artb_bm_alloc(self._h, n, buf) != 0:
            return None
        return list(buf)

    def free(self, blocks: list[int]) -> None:
        if blocks:
            arr = (ctypes.c_int * len(blocks))(*blocks)
            _rt().artb_bm_free(self._h, arr, len(blocks))

    def match_prefix(self, tokens: list[int], salt: int) -> list[int]:
        n = len(tokens)
        max_out = n // self.block_size
        if max_out == 0:
            return []
        tok = (ctypes.c_int32 * n)(*tokens)
        out = (ctypes.c_int * max_out)()
        m = _rt().artb_bm_match_prefix(self._h, tok, n, ctypes.c_uint64(salt & (2 ** 64 - 1)), out, max_out)
        return list(out[:m])

    def commit(self, blocks: list[int], tokens: list[int], salt: int) -> None:
        n_full = min(len(blocks), len(tokens) // self.block_size)
        if n_full <= 0:
            return
        arr = (ctypes.c_int * n_full)(*blocks[:n_full])
        tok = (ctypes.c_int32 * len(tokens))(*tokens)
        _rt().artb_bm_commit(self._h, arr, n_full, tok, len(tokens), ctypes.c_uint64(salt & (2 ** 64 - 1)))

    def reset_prefix_cache(self) -> None:
        _rt().artb_bm_reset_cache(self._h)

    def stats(self) -> dict[str, int]:
        out = (ctypes.c_uint64 * 4)()
        _rt().artb_bm_stats(self._h, out)
        return {"prefix_queries": out[0], "prefix_hits": out[1], "free_blocks": out[2], "cached_free_blocks": out[3]}


class _DevMem:
    """``__cuda_array_interface__`` carrier so torch can view arena memory."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class VmmArena:
    """Reserved virtual address range whose physical backing can be mapped / unmapped (``csrc/kernels/kv_arena.cu``)."""

    def __init__(self, nbytes: int, device: torch.device, chunk_bytes: int = 64 << 20):
        lib = _lib.kernels()
        vp, sz = ctypes.c_void_p, ctypes.c_size_t
        lib.artb_arena_create.argtypes, lib.artb_arena_create.restype = [sz, sz], vp
        lib.artb_arena_base.argtypes, lib.artb_arena_base.restype = [vp], ctypes.c_uint64
        lib.artb_arena_reserved.argtypes, lib.artb_arena_reserved.restype = [vp], sz
        lib.artb_arena_mapped_bytes.argtypes, lib.artb_arena_mapped_bytes.restype = [vp], sz
        lib.artb_arena_map.argtypes, lib.artb_arena_map.restype = [vp, sz, sz], ctypes.c_int
        lib.artb_arena_unmap.argtypes, lib.artb_arena_unmap.restype = [vp, sz, sz], ctypes.c_int
        lib.artb_arena_destroy.argtypes = [vp]
        self._lib, self.device = lib, torch.device(device)
        with torch.cuda.device(self.device):
            self._h = lib.artb_arena_create(nbytes, chunk_bytes)
        if not self._h:
            raise RuntimeError("virtual-memory arena unavailable on this device / driver")
        self.base = int(lib.artb_arena_base(self._h))
        self.reserved = int(lib.artb_arena_reserved(self._h))

    @property
    def mapped_bytes(self) -> int:
        return int(self._lib.artb_arena_mapped_bytes(self._h))

    def map(self, offset: int = 0, nbytes: int | None = None) -> None:
        with torch.cuda.device(self.device):
            _lib.check_rc(self._lib.artb_arena_map(self._h, offset, self.reserved - offset if nbytes is None else nbytes),
                          "arena_map")

    def unmap(self, offset: int = 0, nbytes: int | None = None) -> None:
        torch.cuda.synchronize(self.device)
        with torch.cuda.device(self.device):
            _lib.check_rc(self._lib.artb_arena_unmap(self._h, offset, self.reserved - offset if nbytes is None else nbytes),
                          "arena_unmap")

    def tensor(self, offset: int, shape: tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for d in shape:
            n *= d
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        if offset + nbytes > self.reserved:
            raise ValueError("view outside the arena")
        raw = torch.as_tensor(_DevMem(self.base + offset, nbytes), device=self.device)
        return raw.view(dtype).view(*shape)

    def close(self) -> None:
        h, self._h = self._h, None
        if h:
            self._lib.artb_arena_destroy(h)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class KVCache:
    """Device tensors of the paged cache, one (k, v) pair per layer.

    With ``use_arena`` the tensors live in a :class:`VmmArena`: ``discard`` / ``offload`` hand the physical memory back
    to the driver while every tensor keeps its address, so block tables, captured CUDA graphs and kernel arguments that
    point into the cache stay valid across a sleep / wake cycle.
    """

    def __init__(self, num_layers: int, num_blocks: int, block_size: int, num_kv_heads: int, head_dim: int,
                 device: torch.device, dtype: torch.dtype = torch.bfloat16, use_arena: bool = False):
        self.shape = (num_blocks, block_size, num_kv_heads, head_dim)
        self.device, self.dtype, self.num_layers = device, dtype, num_layers
        self.k: list[torch.Tensor] = []
        self.v: list[torch.Tensor] = []
        self._host: list[tuple[torch.Tensor, torch.Tensor]] | None = None
        self.arena: VmmArena | None = None
        self._views: tuple[list[torch.Tensor], list[torch.Tensor]] | None = None
        if use_arena and torch.device(device).type == "cuda":
            per = num_blocks * block_size * num_kv_heads * head_dim * torch.empty((), dtype=dtype).element_size()
            per = (per + 255) // 256 * 256
            self.arena = VmmArena(2 * num_layers * per, device)
            self.arena.map()     # views can only be created over mapped memory; they stay valid across unmap / map
            self._views = ([self.arena.tensor((2 * i) * per, self.shape, dtype) for i in range(num_layers)],
                           [self.arena.tensor((2 * i + 1) * per, self.shape, dtype) for i in range(num_layers)])
        self._allocate()

    def _allocate(self) -> None:
        if self.arena is not None:
            self.arena.map()
            self.k, self.v = list(self._views[0]), list(self._views[1])
            for t in self.k + self.v:
                t.zero_()
            return
        self.k = [torch.zeros(self.shape, dtype=self.dtype, device=self.device) for _ in range(self.num_layers)]
        self.v = [torch.zeros(self.shape, dtype=self.dtype, device=self.device) for _ in range(self.num_layers)]

    @staticmethod
    def bytes_per_block(num_layers: int, block_size: int, num_kv_heads: int, head_dim: int, elem: int = 2) -> int:
        return 2 * num_layers * block_size * num_kv_heads * head_dim * elem

    @property
    def resident(self) -> bool:
        return bool(self.k)

    def discard(self) -> None:
        """Sleep level 2: free the device memory, contents are lost."""
        self.k, self.v, self._host = [], [], None
        if self.arena is not None:
            self.arena.unmap()
        elif self.device.type == "cuda":
            torch.cuda.empty_cache()

    def offload(self) -> None:
        """Sleep level 1: copy to pinned host memory and free the device memory."""
        pin = self.device.type == "cuda"
        self._host = [(k.to("cpu", non_blocking=False).pin_memory() if pin else k.clone(),
                       v.to("cpu", non_blocking=False).pin_memory() if pin else v.clone())
                      for k, v in zip(self.k, self.v)]
        self.k, self.v = [], []
        if self.arena is not None:
            self.arena.unmap()
        elif pin:
            torch.cuda.empty_cache()

    def restore(self) -> None:
        if self.resident:
            return
        if self._host is None:
            self._allocate()
            return
        if self.arena is not None:
            self.arena.map()
            self.k, self.v = list(self._views[0]), list(self._views[1])
            for (hk, hv), k, v in zip(self._host, self.k, self.v):
                k.copy_(hk, non_blocking=True)
                v.copy_(hv, non_blocking=True)
            self._host = None
            return
        self.k = [k.to(self.device, non_blocking=True) for k, _ in self._host]
        self.v = [v.to(self.device, non_blocking=True) for _, v in self._host]
        self._host = None
