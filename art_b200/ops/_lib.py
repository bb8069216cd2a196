"""ctypes binding to the in-tree native libraries.

The CUDA kernels are exported with a C ABI (``artb_*`` symbols in
``art_b200/_native/libartb_kernels.so``) and take raw device pointers plus the
CUDA stream, so a call is: check shapes in Python, pass ``tensor.data_ptr()`` and
``torch.cuda.current_stream().cuda_stream``.  There is no fallback: if a CUDA
device is present and the library cannot be loaded, importing an op raises.

Every kernel that can wait on something (an mbarrier, a peer's flag) does so with
a bounded number of polls and reports expiry through a per-device int32 status
word; :func:`check_status` reads it (one device sync) and raises
:class:`KernelStatusError`.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

import torch

_NATIVE = Path(__file__).resolve().parent.parent / "_native"
_lock = threading.Lock()
_kernels: ctypes.CDLL | None = None
_runtime: ctypes.CDLL | None = None
_status: dict[int, torch.Tensor] = {}

STATUS_NAMES = {
    0: "ok",
    1: "timeout waiting for a TMA stage",
    2: "timeout waiting for a free smem stage",
    3: "timeout waiting for a TMEM accumulator",
    4: "timeout waiting for a drained TMEM accumulator",
    5: "timeout waiting for a peer rank's flag",
    6: "bad kernel arguments",
    7: "dispatch buffer overflow",
    8: "index outside its buffer (checked build; the access was skipped)",
}


class NativeLibraryError(RuntimeError):
    pass


class KernelStatusError(RuntimeError):
    def __init__(self, code: int):
        super().__init__(f"kernel reported status {code}: {STATUS_NAMES.get(code, 'unknown')}")
        self.code = code


def _load(name: str) -> ctypes.CDLL:
    path = _NATIVE / name
    if not path.exists():
        # Build on demand where a compiler is available (developer machines, CI).
        from .. import build as _build

        try:
            _build.build_all(checked=name.endswith("_checked.so"))
        except Exception as e:  # pragma: no cover - depends on toolchain
            raise NativeLibraryError(f"{path} is missing and could not be built: {e}") from e
    try:
        return ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)
    except OSError as e:
        raise NativeLibraryError(f"cannot load {path}: {e}") from e


def kernels() -> ctypes.CDLL:
    """The CUDA kernel library (requires a CUDA runtime to load)."""
    global _kernels
    if _kernels is None:
        with _lock:
            if _kernels is None:
                # ARTB_BOUNDS_CHECK=1: the build with device-side index checks (python -m art_b200.build --checked);
                # a missing library is an error, never a silent switch back to the unchecked one
                _kernels = _load("libartb_kernels_checked.so" if bounds_checked() else "libartb_kernels.so")
    return _kernels


def bounds_checked() -> bool:
    """True when this process runs the kernel library that was compiled with index checks."""
    return os.environ.get("ARTB_BOUNDS_CHECK", "0") not in ("", "0")


def runtime() -> ctypes.CDLL:
    """The host runtime library (pure C++, loads anywhere)."""
    global _runtime
    if _runtime is None:
        with _lock:
            if _runtime is None:
                _runtime = _load("libartb_runtime.so")
    return _runtime


def have_cuda_kernels() -> bool:
    return torch.cuda.is_available()


def stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def status_word(device: torch.device | int | None = None) -> torch.Tensor:
    idx = torch.cuda.current_device() if device is None else torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    if idx not in _status:
        _status[idx] = torch.zeros(4, dtype=torch.int32, device=f"cuda:{idx}")
    return _status[idx]


def check_status(device: torch.device | int | None = None, reset: bool = True) -> None:
    """Raise if any kernel on ``device`` recorded a bounded-wait expiry since the last check."""
    word = status_word(device)
    code = int(word[0].item())
    if code != 0:
        if reset:
            word.zero_()
        raise KernelStatusError(code)


LAUNCHES = 0  # native kernel launches issued by this process (each front-end call checks its return code once)


def check_rc(rc: int, what: str) -> None:
    global LAUNCHES
    if rc == 0:
        LAUNCHES += 1
        return
    if rc < 0:
        names = {-1: "bad shape", -2: "bad alignment", -3: "driver entry point unavailable",
                 -4: "tensor-map encoding failed", -5: "size beyond the supported maximum"}
        raise ValueError(f"{what}: {names.get(rc, rc)}")
    raise RuntimeError(f"{what}: CUDA error {rc}")


def _env_flag(name: str, default: bool) -> bool:
    v = os.environ.get(name)
    if v is None:
        return default
    return v not in ("0", "false", "False", "")
