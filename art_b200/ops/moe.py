"""Mixture-of-experts ops: router, expert-sorted row plan, gather / combine, grouped GEMM, grouped
LoRA gradient (``csrc/kernels/moe.cu``, ``gemm_grouped.cu``, ``lora_wgrad.cu``).

All data-dependent sizes stay on the device: buffers are sized for the worst case
(``M * k + E * 127`` rows, rounded to 128) and the kernels read the real extent from
``seg_off[E]`` / ``tile_expert``; nothing here synchronises with the host.

The reference handles dense models only; ``reference_*`` are the fp32 PyTorch restatements used
by the tests.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _lib
from .gemm import EPI_BF16, EPI_SWIGLU

_configured = False


def _k():
    global _configured
    lib = _lib.kernels()
    if not _configured:
        vp, ci, cl = ctypes.c_void_p, ctypes.c_int, ctypes.c_long
        lib.artb_moe_router.argtypes = [vp, ci, ci, ci, ci, ci, vp, vp, vp, vp]
        lib.artb_moe_plan.argtypes = [vp, ci, vp, vp, cl, ci, vp, vp, ci, vp, vp, vp, vp, vp]
        lib.artb_moe_gather.argtypes = [vp, ci, vp, vp, ci, vp, vp, ci, ci, ci, vp]
        lib.artb_moe_combine.argtypes = [vp, ci, vp, vp, ci, ci, vp, ci, vp, ci, ci, vp, ci, vp, vp]
        lib.artb_moe_router_bwd.argtypes = [vp, ci, vp, vp, vp, ci, ci, ci, ci, vp, ci, vp]
        lib.artb_gemm_grouped_bf16_tn.argtypes = [vp, ci, vp, ci, vp, ci, vp, ci, ci, vp, ci, vp, ci, vp, ci, ci, ci,
                                                  ci, ci, vp, vp]
        lib.artb_lora_wgrad_grouped.argtypes = [vp, ci, vp, ci, vp, ci, cl, vp, ci, ci, ci, ci, vp]
        for f in (lib.artb_moe_router, lib.artb_moe_plan, lib.artb_moe_gather, lib.artb_moe_combine,
                  lib.artb_moe_router_bwd, lib.artb_gemm_grouped_bf16_tn, lib.artb_lora_wgrad_grouped):
            f.restype = ci
        _configured = True
    return lib


@dataclass
class RoutePlan:
    """Routing decision of one MoE layer for M tokens (everything on the device)."""
    M: int
    k: int
    E: int
    cap_tiles: int
    topi: torch.Tensor        # int32 [M, k]
    topw: torch.Tensor        # fp32  [M, k]
    counts: torch.Tensor      # int32 [E]
    seg_off: torch.Tensor     # int32 [E + 1]   padded segment offsets (multiples of 128)
    tile_expert: torch.Tensor  # int32 [cap_tiles]
    pos: torch.Tensor         # int32 [M, k]    row of (token, slot) in the expert-sorted order
    row_token: torch.Tensor   # int32 [cap_rows] token of each row, -1 for padding
    row_w: torch.Tensor       # fp32  [cap_rows]

    @property
    def cap_rows(self) -> int:
        return self.cap_tiles * 128

    @property
    def total_rows(self) -> torch.Tensor:
        return self.seg_off[self.E:self.E + 1]


def cap_tiles_for(M: int, k: int, E: int) -> int:
    return (M * k + E * 127 + 127) // 128


def route(logits: torch.Tensor, k: int, norm_topk: bool) -> RoutePlan:
    """Softmax over experts, top-k, (optional) renormalisation, and the expert-sorted row plan."""
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    M, E = logits.shape
    dev = logits.device
    i32 = dict(dtype=torch.int32, device=dev)
    cap = cap_tiles_for(M, k, E)
    plan = RoutePlan(M, k, E, cap, torch.empty((M, k), **i32), torch.empty((M, k), dtype=torch.float32, device=dev),
                     torch.zeros(E, **i32), torch.empty(E + 1, **i32), torch.empty(cap, **i32),
                     torch.empty((M, k), **i32), torch.empty(cap * 128, **i32),
                     torch.empty(cap * 128, dtype=torch.float32, device=dev))
    cursor = torch.empty(E, **i32)
    st = _lib.stream_ptr()
    _lib.check_rc(_k().artb_moe_router(_lib.ptr(logits), logits.stride(0), M, E, k, int(norm_topk), _lib.ptr(plan.topi),
                                       _lib.ptr(plan.topw), _lib.ptr(plan.counts), st), "moe_router")
    _lib.check_rc(_k().artb_moe_plan(_lib.ptr(plan.counts), E, _lib.ptr(plan.topi), _lib.ptr(plan.topw), M, k,
                                     _lib.ptr(plan.seg_off), _lib.ptr(plan.tile_expert), cap, _lib.ptr(cursor),
                                     _lib.ptr(plan.pos), _lib.ptr(plan.row_token), _lib.ptr(plan.row_w), st),
                  "moe_plan")
    return plan


def gather(x: torch.Tensor, plan: RoutePlan, weighted: bool = False, out: torch.Tensor | None = None) -> torch.Tensor:
    """``xp[row] = x[token(row)]`` (times the routing weight if ``weighted``); padding rows are zero."""
    D = x.shape[1]
    if out is None:
        out = torch.empty((plan.cap_rows, D), dtype=torch.bfloat16, device=x.device)
    _lib.check_rc(_k().artb_moe_gather(_lib.ptr(x), x.stride(0), _lib.ptr(plan.row_token), _lib.ptr(plan.row_w),
                                       int(weighted), _lib.ptr(plan.total_rows), _lib.ptr(out), out.stride(0), D,
                                       plan.cap_rows, _lib.stream_ptr()), "moe_gather")
    return out


def combine(yp: torch.Tensor, plan: RoutePlan, weighted: bool = True, residual: torch.Tensor | None = None,
            out: torch.Tensor | None = None, grad_for_dots: torch.Tensor | None = None,
            want_out: bool = True) -> tuple[torch.Tensor | None, torch.Tensor | None]:
    """``out[t] = residual[t] + sum_s w[t,s] * yp[pos[t,s]]``; with ``grad_for_dots`` also returns
    ``dots[t,s] = <grad[t], yp[pos[t,s]]>`` (the gradient of the routing weights)."""
    D = yp.shape[1]
    if want_out and out is None:
        out = torch.empty((plan.M, D), dtype=torch.bfloat16, device=yp.device)
    dots = None
    if grad_for_dots is not None:
        dots = torch.empty((plan.M, plan.k), dtype=torch.float32, device=yp.device)
    _lib.check_rc(_k().artb_moe_combine(
        _lib.ptr(yp), yp.stride(0), _lib.ptr(plan.pos), _lib.ptr(plan.topw if weighted else None), plan.M, plan.k,
        _lib.ptr(residual), residual.stride(0) if residual is not None else 0,
        _lib.ptr(out if want_out else None), out.stride(0) if want_out else 0, D,
        _lib.ptr(grad_for_dots), grad_for_dots.stride(0) if grad_for_dots is not None else 0, _lib.ptr(dots),
        _lib.stream_ptr()), "moe_combine")
    return (out if want_out else None), dots


def router_bwd(logits: torch.Tensor, plan: RoutePlan, dw: torch.Tensor, norm_topk: bool, ld_out: int) -> torch.Tensor:
    """bf16 ``dlogits [M, ld_out]`` (columns >= E zero) from the gradient of the top-k weights."""
    M, E = logits.shape
    out = torch.empty((M, ld_out), dtype=torch.bfloat16, device=logits.device)
    _lib.check_rc(_k().artb_moe_router_bwd(_lib.ptr(logits), logits.stride(0), _lib.ptr(plan.topi), _lib.ptr(plan.topw),
                                           _lib.ptr(dw), M, E, plan.k, int(norm_topk), _lib.ptr(out), out.stride(0),
                                           _lib.stream_ptr()), "moe_router_bwd")
    return out


def grouped_gemm(a: torch.Tensor, b: torch.Tensor, plan: RoutePlan, n_per_expert: int, a2: torch.Tensor | None = None,
                 b2: torch.Tensor | None = None, swiglu_out: torch.Tensor | None = None,
                 out: torch.Tensor | None = None) -> torch.Tensor:
    """``out[rows of e] = a[rows of e] @ b[e*N:(e+1)*N].T (+ a2[rows] @ b2[e*N:(e+1)*N].T)``."""
    rows, K = a.shape
    assert rows == plan.cap_rows and b.shape == (plan.E * n_per_expert, K)
    if out is None:
        out = torch.empty((rows, n_per_expert), dtype=torch.bfloat16, device=a.device)
    K2 = a2.shape[1] if a2 is not None else 0
    rc = _k().artb_gemm_grouped_bf16_tn(
        _lib.ptr(a), a.stride(0), _lib.ptr(b), b.stride(0), _lib.ptr(a2), a2.stride(0) if a2 is not None else 0,
        _lib.ptr(b2), b2.stride(0) if b2 is not None else 0, K2, _lib.ptr(out), out.stride(0),
        _lib.ptr(swiglu_out), swiglu_out.stride(0) if swiglu_out is not None else 0, _lib.ptr(plan.tile_expert),
        plan.cap_tiles, plan.E, n_per_expert, K, EPI_SWIGLU if swiglu_out is not None else EPI_BF16,
        _lib.ptr(_lib.status_word(a.device)), _lib.stream_ptr())
    _lib.check_rc(rc, "gemm_grouped")
    return out


def grouped_wgrad(acc: torch.Tensor, p: torch.Tensor, q: torch.Tensor, plan: RoutePlan, splits: int = 2) -> None:
    """``acc[e] [C, 64] += p[rows of e].T @ q[rows of e]`` for every expert (fp32 accumulation)."""
    E, C, R = acc.shape
    assert R == 64 and q.shape[1] == 64 and p.shape[1] == C and acc.is_contiguous()
    _lib.check_rc(_k().artb_lora_wgrad_grouped(_lib.ptr(p), p.stride(0), _lib.ptr(q), q.stride(0), _lib.ptr(acc), R,
                                               C * R, _lib.ptr(plan.seg_off), E, C, splits, min(p.shape[0], q.shape[0]),
                                               _lib.stream_ptr()),
                  "lora_wgrad_grouped")


# ------------------------------------------------------------------------------------ references
def reference_route(logits: torch.Tensor, k: int, norm_topk: bool) -> tuple[torch.Tensor, torch.Tensor]:
    probs = logits.float().softmax(-1)
    topw, topi = probs.topk(k, dim=-1)
    if norm_topk:
        topw = topw / topw.sum(-1, keepdim=True)
    return topi, topw
