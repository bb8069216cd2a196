"""Tree-masked attention over packed rows.

Tokens of several packed rows are laid out back to back: ``qkv`` is ``[M, (Hq + 2*Hkv) * hd]``
with ``M = rows * S``.  A query may attend a key of the same row iff
``k <= q and (group[q] == group[k] or parent[q] == group[k])``
(reference mask: ``src/art/local/train.py:177-215``, there materialised as a dense
``[B,S,S]`` bias; here evaluated from the two id vectors).

``impl="native"`` runs the flash-style kernels of ``csrc/kernels/attn_tree.cu`` (mask from
ids per tile, fully-masked tiles skipped); ``impl="sdpa"`` is the library baseline, which
builds the dense mask and calls ``scaled_dot_product_attention``.  An :class:`AttnPlan` is
made once per micro-batch and shared by all layers, forward and backward.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F


@dataclass
class AttnPlan:
    impl: str
    gid: torch.Tensor   # int32 [M]
    pid: torch.Tensor   # int32 [M]
    S: int
    state: torch.Tensor | None = None   # native: uint8 tile states
    mask: torch.Tensor | None = None    # sdpa: dense bool mask [rows,1,S,S]


@dataclass
class AttnCtx:
    plan: AttnPlan
    saved: tuple


def dense_mask(gid: torch.Tensor, pid: torch.Tensor) -> torch.Tensor:
    """[R,S] ids -> bool [R,S,S]."""
    S = gid.shape[-1]
    causal = torch.ones(S, S, dtype=torch.bool, device=gid.device).tril()
    return causal & ((gid.unsqueeze(2) == gid.unsqueeze(1)) | (pid.unsqueeze(2) == gid.unsqueeze(1)))


def make_plan(gid: torch.Tensor, pid: torch.Tensor, S: int, impl: str = "native") -> AttnPlan:
    plan = AttnPlan(impl, gid, pid, S)
    if impl == "native":
        from . import attn_native

        if S % 64:
            raise ValueError("native attention needs the packed row length to be a multiple of 64")
        plan.state = attn_native.tile_states(gid, pid, S)
    else:
        rows = gid.numel() // S
        plan.mask = dense_mask(gid.view(rows, S), pid.view(rows, S)).unsqueeze(1)
    return plan


def _split(qkv: torch.Tensor, rows: int, S: int, Hq: int, Hkv: int, hd: int):
    q = qkv[:, : Hq * hd].reshape(rows, S, Hq, hd).transpose(1, 2)
    k = qkv[:, Hq * hd: (Hq + Hkv) * hd].reshape(rows, S, Hkv, hd).transpose(1, 2)
    v = qkv[:, (Hq + Hkv) * hd:].reshape(rows, S, Hkv, hd).transpose(1, 2)
    return q, k, v


def forward(qkv: torch.Tensor, Hq: int, Hkv: int, hd: int, plan: AttnPlan,
            need_grad: bool = True) -> tuple[torch.Tensor, AttnCtx]:
    M, S = qkv.shape[0], plan.S
    rows = M // S
    if plan.impl == "native":
        from . import attn_native

        o, saved = attn_native.forward(qkv, Hq, Hkv, hd, plan)
        return o, AttnCtx(plan, saved)
    q, k, v = _split(qkv, rows, S, Hq, Hkv, hd)
    if need_grad:
        q, k, v = (t.detach().requires_grad_(True) for t in (q, k, v))
    with torch.enable_grad() if need_grad else torch.no_grad():
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=plan.mask, enable_gqa=(Hq != Hkv))
        o2 = o.transpose(1, 2).reshape(M, Hq * hd)
    return o2.detach(), AttnCtx(plan, (q, k, v, o2))


def backward(do: torch.Tensor, ctx: AttnCtx) -> torch.Tensor:
    """Gradient w.r.t. the fused post-RoPE ``qkv`` buffer, same layout."""
    if ctx.plan.impl == "native":
        from . import attn_native

        return attn_native.backward(do, ctx.saved, ctx.plan)
    q, k, v, o2 = ctx.saved
    dq, dk, dv = torch.autograd.grad(o2, (q, k, v), do)
    M = do.shape[0]
    return torch.cat([dq.transpose(1, 2).reshape(M, -1), dk.transpose(1, 2).reshape(M, -1),
                      dv.transpose(1, 2).reshape(M, -1)], dim=1)


def reference(qkv, Hq, Hkv, hd, gid, pid, S):
    """fp32 dense restatement: returns o [M, Hq*hd]."""
    M = qkv.shape[0]
    rows = M // S
    q, k, v = (t.float() for t in _split(qkv, rows, S, Hq, Hkv, hd))
    rep = Hq // Hkv
    k = k.repeat_interleave(rep, 1)
    v = v.repeat_interleave(rep, 1)
    s = q @ k.transpose(-1, -2) / math.sqrt(hd)
    s = s.masked_fill(~dense_mask(gid.view(rows, S), pid.view(rows, S)).unsqueeze(1), float("-inf"))
    return (s.softmax(-1) @ v).transpose(1, 2).reshape(M, Hq * hd)
