"""LoRA factor-gradient accumulation ``acc[C, 64] += p[M, C].T @ q[M, 64]``
(``csrc/kernels/lora_wgrad.cu``)."""
from __future__ import annotations

import ctypes

import torch

from . import _lib

_fn = None


def accumulate(acc: torch.Tensor, p: torch.Tensor, q: torch.Tensor, transpose_out: bool = False) -> None:
    """``acc`` fp32 [C, R]; ``p`` bf16 [M, C] (the wide operand); ``q`` bf16 [M, R], R == 64.

    ``transpose_out`` is accepted for call-site readability only: both LoRA gradients are
    stored with the wide dimension first, so the arithmetic is identical.
    """
    global _fn
    if not p.is_cuda:
        acc.add_(p.float().t() @ q.float())
        return
    M, C = p.shape
    R = q.shape[1]
    if R != 64:
        for c in range(0, R, 64):
            accumulate(acc[:, c:c + 64], p, q[:, c:c + 64])
        return
    if _fn is None:
        _fn = _lib.kernels().artb_lora_wgrad
        vp, ci = ctypes.c_void_p, ctypes.c_int
        _fn.argtypes = [vp, ci, vp, ci, vp, ci, ci, ci, vp]
        _fn.restype = ci
    assert acc.dtype == torch.float32 and acc.stride(1) == 1 and acc.shape[0] == C
    _lib.check_rc(_fn(_lib.ptr(p), p.stride(0), _lib.ptr(q), q.stride(0), _lib.ptr(acc), acc.stride(0), M, C,
                      _lib.stream_ptr()), "lora_wgrad")
