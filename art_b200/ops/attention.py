"""Tree-masked attention over packed rows.

Tokens of several packed rows are laid out back to back: ``qkv`` is ``[M, (Hq + 2*Hkv) * hd]``
with ``M = rows * S``.  A query may attend a key of the same row iff
``k <= q and (group[q] == group[k] or parent[q] == group[k])``
(reference mask: ``src/art/local/train.py:177-215``, there materialised as a dense
``[B,S,S]`` bias; here evaluated from the two id vectors).

``impl="native"`` runs the flash-style kernels of ``csrc/kernels/attn_tree.cu`` (mask from
ids per tile, fully-masked tiles skipped); ``impl="sdpa"`` is the library baseline, which
builds the dense mask and calls ``scaled_dot_product_attention``.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import _lib


@dataclass
class AttnCtx:
    impl: str
    saved: tuple


def dense_mask(gid: torch.Tensor, pid: torch.Tensor) -> torch.Tensor:
    """[R,S] ids -> bool [R,S,S]."""
    S = gid.shape[-1]
    causal = torch.ones(S, S, dtype=torch.bool, device=gid.device).tril()
    return causal & ((gid.unsqueeze(2) == gid.unsqueeze(1)) | (pid.unsqueeze(2) == gid.unsqueeze(1)))


def _split(qkv: torch.Tensor, rows: int, S: int, Hq: int, Hkv: int, hd: int):
    q = qkv[:, : Hq * hd].reshape(rows, S, Hq, hd).transpose(1, 2)
    k = qkv[:, Hq * hd: (Hq + Hkv) * hd].reshape(rows, S, Hkv, hd).transpose(1, 2)
    v = qkv[:, (Hq + Hkv) * hd:].reshape(rows, S, Hkv, hd).transpose(1, 2)
    return q, k, v


def forward(qkv: torch.Tensor, Hq: int, Hkv: int, hd: int, gid: torch.Tensor, pid: torch.Tensor, S: int,
            impl: str = "native", need_grad: bool = True) -> tuple[torch.Tensor, AttnCtx]:
    M = qkv.shape[0]
    rows = M // S
    if impl == "native":
        from . import attn_native

        return attn_native.forward(qkv, Hq, Hkv, hd, gid, pid, S, need_grad)
    q, k, v = _split(qkv, rows, S, Hq, Hkv, hd)
    if need_grad:
        q, k, v = (t.detach().requires_grad_(True) for t in (q, k, v))
    mask = dense_mask(gid.view(rows, S), pid.view(rows, S)).unsqueeze(1)
    with torch.enable_grad() if need_grad else torch.no_grad():
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=mask, enable_gqa=(Hq != Hkv))
        o2 = o.transpose(1, 2).reshape(M, Hq * hd)
    return o2.detach(), AttnCtx("sdpa", (q, k, v, o2))


def backward(do: torch.Tensor, ctx: AttnCtx) -> torch.Tensor:
    """Gradient w.r.t. the fused post-RoPE ``qkv`` buffer, same layout."""
    if ctx.impl == "native":
        from . import attn_native

        return attn_native.backward(do, ctx)
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
