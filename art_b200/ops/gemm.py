"""tcgen05 GEMM front-end: ``C = A @ B.T (+ A2 @ B2.T)`` with fused epilogues.

The kernel lives in ``csrc/kernels/gemm_tcgen05.cu``; this module validates
shapes/strides and passes raw pointers.  ``reference_gemm_tn`` is the fp32
PyTorch restatement used by the tests.
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import _lib

EPI_BF16, EPI_BF16_RESID, EPI_F32, EPI_SWIGLU, EPI_SWIGLU_BWD = 0, 1, 2, 3, 4
_configured = False
_configured2 = False
TWO_CTA_DEFAULT = os.environ.get("ARTB_GEMM_2CTA", "1") == "1"


def _fn():
    global _configured
    f = _lib.kernels().artb_gemm_bf16_tn
    if not _configured:
        vp, ci = ctypes.c_void_p, ctypes.c_int
        f.argtypes = [vp, ci, vp, ci, vp, ci, vp, ci, ci, vp, ci, vp, ci, vp, ci, vp, ci, ci, ci, ci, ci, ci, vp, ci, vp]
        f.restype = ci
        _configured = True
    return f


def _fn2():
    global _configured2
    f = _lib.kernels().artb_gemm_bf16_tn_2cta
    if not _configured2:
        vp, ci = ctypes.c_void_p, ctypes.c_int
        f.argtypes = [vp, ci, vp, ci, vp, ci, vp, ci, ci, vp, ci, vp, ci, vp, ci, vp, ci, ci, ci, ci, ci, vp, ci, vp]
        f.restype = ci
        _configured2 = True
    return f


def _check2d(t: torch.Tensor, name: str) -> None:
    if t.dim() != 2 or t.dtype != torch.bfloat16 or not t.is_cuda or t.stride(1) != 1:
        raise ValueError(f"{name}: expected a 2-D bf16 CUDA tensor with unit inner stride, got "
                         f"{tuple(t.shape)} {t.dtype} strides {t.stride()}")


def gemm_tn(a: torch.Tensor, b: torch.Tensor, *, a2: torch.Tensor | None = None,
            b2: torch.Tensor | None = None, out: torch.Tensor | None = None,
            residual: torch.Tensor | None = None, swiglu_out: torch.Tensor | None = None,
            bias: torch.Tensor | None = None, res_cols: int = 0,
            out_dtype: torch.dtype = torch.bfloat16, bn: int = 0, max_ctas: int = 0,
            two_cta: bool | None = None, swiglu_bwd_gu: torch.Tensor | None = None) -> torch.Tensor:
    """``out[M,N] = a[M,K] @ b[N,K].T (+ a2[M,K2] @ b2[N,K2].T) (+ residual)``.

    ``swiglu_out`` ([M, N/2] bf16) selects the SwiGLU epilogue: ``b``'s rows must be
    interleaved in blocks of 16 (gate rows, then the matching up rows); ``out`` receives
    the pre-activation and ``swiglu_out`` receives ``silu(gate) * up``.

    ``swiglu_bwd_gu`` ([M, 2N] bf16, the forward's interleaved gate|up pre-activations) selects the fused
    SwiGLU-backward epilogue: the product is taken as ``d(silu(gate) * up)`` and ``out`` ([M, 2N]) receives
    ``d(gate|up)`` in the same interleaved layout; the activation gradient itself is never written.
    """
    _check2d(a, "a")
    _check2d(b, "b")
    M, K = a.shape
    N, Kb = b.shape
    if K != Kb:
        raise ValueError(f"K mismatch: {K} vs {Kb}")
    K2 = 0
    if a2 is not None:
        _check2d(a2, "a2")
        _check2d(b2, "b2")
        K2 = a2.shape[1]
        if a2.shape[0] != M or b2.shape[0] != N or b2.shape[1] != K2:
            raise ValueError("extra-K operands must be [M,K2] and [N,K2]")
    if swiglu_bwd_gu is not None:
        _check2d(swiglu_bwd_gu, "swiglu_bwd_gu")
        if tuple(swiglu_bwd_gu.shape) != (M, 2 * N) or N % 32:
            raise ValueError("swiglu_bwd_gu must be [M, 2N] with N a multiple of 32")
        if out is None:
            out = torch.empty((M, 2 * N), dtype=torch.bfloat16, device=a.device)
        epi = EPI_SWIGLU_BWD
        swiglu_out = swiglu_bwd_gu          # travels in the H slot of the C entry point
    elif swiglu_out is not None:
        epi = EPI_SWIGLU
    elif residual is not None:
        epi = EPI_BF16_RESID
    elif out_dtype == torch.float32:
        epi = EPI_F32
    else:
        epi = EPI_BF16
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32 if epi == EPI_F32 else torch.bfloat16, device=a.device)
    if out.stride(1) != 1 or tuple(out.shape) != (M, 2 * N if epi == EPI_SWIGLU_BWD else N):
        raise ValueError("out must be [M,N] with unit inner stride")
    if residual is not None:
        _check2d(residual, "residual")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise ValueError("bias must be fp32 [N]")
    st = _lib.status_word(a.device)
    if two_cta is None:
        two_cta = TWO_CTA_DEFAULT and bn == 0 and M >= 1024 and N >= 512   # bn = 224 with two_cta=True: 256 x 224 pair tiles
    if two_cta:
        rc = _fn2()(
            _lib.ptr(a), a.stride(0), _lib.ptr(b), b.stride(0),
            _lib.ptr(a2), a2.stride(0) if a2 is not None else 0,
            _lib.ptr(b2), b2.stride(0) if b2 is not None else 0, K2,
            _lib.ptr(out), out.stride(0),
            _lib.ptr(residual), residual.stride(0) if residual is not None else 0,
            _lib.ptr(swiglu_out), swiglu_out.stride(0) if swiglu_out is not None else 0,
            _lib.ptr(bias),
            M, N, K, epi, res_cols, _lib.ptr(st), -(max_ctas // 2 or 1 << 20) if bn == 224 else max_ctas // 2,
            _lib.stream_ptr())
        _lib.check_rc(rc, "gemm_tn_2cta")
        return out
    rc = _fn()(
        _lib.ptr(a), a.stride(0), _lib.ptr(b), b.stride(0),
        _lib.ptr(a2), a2.stride(0) if a2 is not None else 0,
        _lib.ptr(b2), b2.stride(0) if b2 is not None else 0, K2,
        _lib.ptr(out), out.stride(0),
        _lib.ptr(residual), residual.stride(0) if residual is not None else 0,
        _lib.ptr(swiglu_out), swiglu_out.stride(0) if swiglu_out is not None else 0,
        _lib.ptr(bias),
        M, N, K, epi, res_cols, bn, _lib.ptr(st), max_ctas, _lib.stream_ptr())
    _lib.check_rc(rc, "gemm_tn")
    return out


def reference_gemm_tn(a, b, a2=None, b2=None, residual=None, bias=None) -> torch.Tensor:
    """fp32 PyTorch restatement (inputs upcast, fp32 accumulation)."""
    c = a.float() @ b.float().t()
    if a2 is not None:
        c = c + a2.float() @ b2.float().t()
    if bias is not None:
        c = c + bias.float()
    if residual is not None:
        c = c + residual.float()
    return c


_sk_configured = False


def gemm_splitk_(ws: torch.Tensor, a: torch.Tensor, b: torch.Tensor, bn: int, splits: int,
                 two_cta: bool = False) -> None:
    """``ws[M, :N] += a @ b.T`` with the K dimension split across CTAs (fp32 atomics); ``ws`` fp32, zero on entry.

    ``two_cta``: 256 x 256 tiles on CTA pairs (``bn`` is ignored); the pair shares every weight tile."""
    global _sk_configured
    f = _lib.kernels().artb_gemm_splitk_bf16_tn
    f2 = _lib.kernels().artb_gemm_splitk_bf16_tn_2cta
    g = _lib.kernels().artb_splitk_finalize
    if not _sk_configured:
        vp, ci = ctypes.c_void_p, ctypes.c_int
        f.argtypes = [vp, ci, vp, ci, vp, ci, ci, ci, ci, ci, ci, vp, vp]
        f.restype = ci
        f2.argtypes = [vp, ci, vp, ci, vp, ci, ci, ci, ci, ci, vp, vp]
        f2.restype = ci
        g.argtypes = [vp, ci, vp, ci, vp, ci, ci, vp, ci, ci, vp, ci, ci, vp]
        g.restype = ci
        _sk_configured = True
    _check2d(a, "a")
    _check2d(b, "b")
    M, K = a.shape
    N = b.shape[0]
    if two_cta:
        rc = f2(_lib.ptr(a), a.stride(0), _lib.ptr(b), b.stride(0), _lib.ptr(ws), ws.stride(0), M, N, K, splits,
                _lib.ptr(_lib.status_word(a.device)), _lib.stream_ptr())
    else:
        rc = f(_lib.ptr(a), a.stride(0), _lib.ptr(b), b.stride(0), _lib.ptr(ws), ws.stride(0), M, N, K, bn, splits,
               _lib.ptr(_lib.status_word(a.device)), _lib.stream_ptr())
    _lib.check_rc(rc, "gemm_splitk")


def splitk_finalize(ws: torch.Tensor, out: torch.Tensor, bias: torch.Tensor | None = None,
                    residual: torch.Tensor | None = None, res_cols: int = 0, adapter: torch.Tensor | None = None,
                    mask_col0: int = 0, cols_per_adapter: int = 0) -> torch.Tensor:
    """``out = bf16(ws[:, :N] + bias + residual)`` and ``ws[:, :N] = 0``.

    With ``adapter`` (int32 [M]) the columns from ``mask_col0`` on are the stacked LoRA shrink products of all
    resident adapters, ``cols_per_adapter`` each: row ``m`` keeps only those of slot ``adapter[m]``."""
    g = _lib.kernels().artb_splitk_finalize
    M, N = out.shape
    rc = g(_lib.ptr(ws), ws.stride(0), _lib.ptr(out), out.stride(0), _lib.ptr(residual),
           residual.stride(0) if residual is not None else 0, res_cols, _lib.ptr(bias), M, N, _lib.ptr(adapter),
           mask_col0, cols_per_adapter, _lib.stream_ptr())
    _lib.check_rc(rc, "splitk_finalize")
    return out


def plan_small_m(M: int, N: int, K: int, sms: int = 148, pair: bool = False) -> tuple[int, int]:
    """(bn, splits) for a weight-streaming GEMM: widest N tile, then split K as far as ONE wave of CTAs allows
    (tiles * splits <= SMs: a second, nearly empty wave would double the time).  ``pair``: 256 x 256 tiles on CTA
    pairs, so the unit is a cluster and there are ``sms // 2`` of them."""
    kb = (K + 63) // 64
    if pair:
        tiles = ((M + 255) // 256) * ((N + 255) // 256)
        if tiles >= 50:
            return 256, 1
        return 256, max(1, min((sms // 2) // tiles, max(1, kb // 4)))
    m_tiles = (M + 127) // 128
    bn = 256 if N >= 256 else (128 if N >= 128 else 64)
    tiles = m_tiles * ((N + bn - 1) // bn)
    if tiles >= 100:
        return bn, 1
    splits = max(1, min(sms // tiles, max(1, kb // 4)))
    return bn, splits


_skinny_ws: dict = {}
SKINNY_SPLITS = int(os.environ.get("ARTB_SKINNY_SPLITS", "4"))


def skinny_gemm(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``out[M, N] = a[M, K] @ b[N, K].T`` for N <= 64 and large M (the LoRA shrink ``X A^T`` and ``dY B``).

    One N tile means only ``M / 128`` CTAs in the plain kernel (64 for 8192 tokens), each streaming all of K, so the
    op is latency-bound; here K is split ``SKINNY_SPLITS`` ways (fp32 atomics into a small zeroed workspace) so the
    whole machine streams ``a`` once, and a finalize pass converts to bf16 and re-zeroes the workspace.
    """
    M, K = a.shape
    N = b.shape[0]
    if N > 64 or M < 2048 or K < 1024 or SKINNY_SPLITS <= 1:
        return gemm_tn(a, b, out=out)
    key = (a.device.index, M, N)
    ws = _skinny_ws.get(key)
    if ws is None:
        ws = _skinny_ws[key] = torch.zeros((M, 64), dtype=torch.float32, device=a.device)
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
    gemm_splitk_(ws, a, b, 64, SKINNY_SPLITS)
    return splitk_finalize(ws, out)
