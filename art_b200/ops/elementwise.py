"""Front-ends for the bandwidth-bound layer kernels in ``csrc/kernels/elementwise.cu``.

Each function has a ``*_reference`` twin in plain fp32 PyTorch used by the numerics tests.
"""
from __future__ import annotations

import ctypes
import json
import math

import torch

from . import _lib

vp, ci, cf, cl = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_long
_sigs = {
    "artb_rmsnorm_fwd": [vp, vp, vp, vp, ci, ci, cf, vp],
    "artb_rmsnorm_bwd": [vp, vp, vp, vp, vp, vp, ci, ci, vp],
    "artb_rope": [vp, vp, ci, ci, ci, ci, ci, cf, ci, vp],
    "artb_rope_table": [vp, vp, ci, ci, ci, ci, ci, vp, cf, ci, vp],
    "artb_swiglu_bwd": [vp, vp, vp, cl, ci, vp],
    "artb_swiglu_fwd": [vp, vp, cl, ci, vp],
    "artb_headnorm_fwd": [vp, vp, vp, ci, ci, ci, ci, ci, cf, vp],
    "artb_headnorm_bwd": [vp, vp, vp, vp, ci, ci, ci, ci, ci, vp],
    "artb_gather_rows": [vp, vp, vp, cl, ci, cl, vp, vp],
    "artb_scatter_rows": [vp, vp, vp, cl, ci, cl, vp, vp],
    "artb_adv_norm": [vp, vp, vp, vp, ci, vp],
}
_bound: dict[str, object] = {}


def _f(name: str):
    fn = _bound.get(name)
    if fn is None:
        fn = getattr(_lib.kernels(), name)
        fn.argtypes = _sigs[name]
        fn.restype = ci
        _bound[name] = fn
    return fn


def rmsnorm_fwd(x: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor | None = None,
                want_rstd: bool = True) -> tuple[torch.Tensor, torch.Tensor | None]:
    M, D = x.shape
    y = torch.empty_like(x) if out is None else out
    rstd = torch.empty(M, dtype=torch.float32, device=x.device) if want_rstd else None
    _lib.check_rc(_f("artb_rmsnorm_fwd")(_lib.ptr(x), _lib.ptr(w), _lib.ptr(y), _lib.ptr(rstd), M, D, eps,
                                         _lib.stream_ptr()), "rmsnorm_fwd")
    return y, rstd


def rmsnorm_bwd(dy: torch.Tensor, x: torch.Tensor, w: torch.Tensor, rstd: torch.Tensor,
                dres: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    M, D = x.shape
    dx = torch.empty_like(x) if out is None else out
    _lib.check_rc(_f("artb_rmsnorm_bwd")(_lib.ptr(dy), _lib.ptr(x), _lib.ptr(w), _lib.ptr(rstd), _lib.ptr(dres),
                                         _lib.ptr(dx), M, D, _lib.stream_ptr()), "rmsnorm_bwd")
    return dx


def rope_(buf: torch.Tensor, pos: torch.Tensor, col0: int, heads: int, hd: int, theta: float,
          inverse: bool = False, freqs: torch.Tensor | None = None, mscale: float = 1.0) -> torch.Tensor:
    """Rotate ``heads`` heads of width ``hd`` starting at column ``col0`` of ``buf`` [M, ld], in place.  ``freqs``
    (fp32 [hd / 2] on the device) replaces ``theta ** (-2 i / hd)`` for frequency-scaled rotary embeddings; ``mscale``
    multiplies cos and sin (see :func:`rope_args`)."""
    assert pos.dtype == torch.int32 and buf.stride(1) == 1
    if freqs is None:
        _lib.check_rc(_f("artb_rope")(_lib.ptr(buf), _lib.ptr(pos), buf.shape[0], buf.stride(0), col0, heads, hd, theta,
                                      1 if inverse else 0, _lib.stream_ptr()), "rope")
    else:
        assert freqs.dtype == torch.float32 and freqs.numel() == hd // 2 and freqs.is_contiguous() and freqs.device == buf.device
        _lib.check_rc(_f("artb_rope_table")(_lib.ptr(buf), _lib.ptr(pos), buf.shape[0], buf.stride(0), col0, heads, hd,
                                            _lib.ptr(freqs), mscale, 1 if inverse else 0,
                                            _lib.stream_ptr()), "rope_table")
    return buf


_rope_tables: dict = {}


def rope_args(cfg, device) -> dict:
    """Keyword arguments of :func:`rope_` for a model configuration: empty for the plain rotation, else the frequency
    table of ``cfg.rope_inv_freq()`` on ``device`` (built once per configuration and device) and the attention scale."""
    if getattr(cfg, "rope_scaling", None) is None:
        return {}
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    key = (cfg.head_dim, cfg.rope_theta, json.dumps(cfg.rope_scaling, sort_keys=True), str(device))
    if key not in _rope_tables:
        inv, att = cfg.rope_inv_freq()
        _rope_tables[key] = {"freqs": torch.tensor(inv, dtype=torch.float32, device=device), "mscale": float(att)}
    return _rope_tables[key]


def swiglu_fwd(gu: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    M, F2 = gu.shape
    h = torch.empty((M, F2 // 2), dtype=gu.dtype, device=gu.device) if out is None else out
    _lib.check_rc(_f("artb_swiglu_fwd")(_lib.ptr(gu), _lib.ptr(h), M, F2 // 2, _lib.stream_ptr()), "swiglu_fwd")
    return h


def swiglu_bwd(dh: torch.Tensor, gu: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    M, F = dh.shape
    dgu = torch.empty_like(gu) if out is None else out
    _lib.check_rc(_f("artb_swiglu_bwd")(_lib.ptr(dh), _lib.ptr(gu), _lib.ptr(dgu), M, F, _lib.stream_ptr()), "swiglu_bwd")
    return dgu


def headnorm_fwd_(buf: torch.Tensor, w: torch.Tensor, col0: int, heads: int, hd: int, eps: float) -> torch.Tensor:
    M = buf.shape[0]
    rstd = torch.empty(M * heads, dtype=torch.float32, device=buf.device)
    _lib.check_rc(_f("artb_headnorm_fwd")(_lib.ptr(buf), _lib.ptr(w), _lib.ptr(rstd), M, buf.stride(0), col0, heads, hd,
                                          eps, _lib.stream_ptr()), "headnorm_fwd")
    return rstd


def headnorm_bwd_(dbuf: torch.Tensor, xbuf: torch.Tensor, w: torch.Tensor, rstd: torch.Tensor, col0: int, heads: int,
                  hd: int) -> None:
    _lib.check_rc(_f("artb_headnorm_bwd")(_lib.ptr(dbuf), _lib.ptr(xbuf), _lib.ptr(w), _lib.ptr(rstd), dbuf.shape[0],
                                          dbuf.stride(0), col0, heads, hd, _lib.stream_ptr()), "headnorm_bwd")


def gather_rows(table: torch.Tensor, idx: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    assert idx.dtype == torch.int64 and table.dtype == torch.bfloat16 and table.is_contiguous()
    n, D = idx.numel(), table.shape[1]
    o = torch.empty((n, D), dtype=table.dtype, device=table.device) if out is None else out
    _lib.check_rc(_f("artb_gather_rows")(_lib.ptr(table), _lib.ptr(idx), _lib.ptr(o), n, D, table.shape[0],
                                         _lib.ptr(_lib.status_word(table.device)), _lib.stream_ptr()), "gather_rows")
    return o


def scatter_rows_(src: torch.Tensor, idx: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    assert idx.dtype == torch.int64 and out.is_contiguous() and src.is_contiguous()
    _lib.check_rc(_f("artb_scatter_rows")(_lib.ptr(src), _lib.ptr(idx), _lib.ptr(out), idx.numel(), out.shape[1],
                                          out.shape[0], _lib.ptr(_lib.status_word(out.device)), _lib.stream_ptr()),
                  "scatter_rows")
    return out


def adv_norm(rewards: torch.Tensor, offsets: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Group-normalised advantages on the device.  ``offsets`` int32 [G+1] CSR boundaries."""
    adv = torch.empty_like(rewards)
    keep = torch.empty(rewards.numel(), dtype=torch.uint8, device=rewards.device)
    _lib.check_rc(_f("artb_adv_norm")(_lib.ptr(rewards), _lib.ptr(offsets), _lib.ptr(adv), _lib.ptr(keep),
                                      offsets.numel() - 1, _lib.stream_ptr()), "adv_norm")
    return adv, keep.bool()


# ------------------------------------------------------------------ fp32 references
def rmsnorm_reference(x, w, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype).float() * w.float()


def rope_reference(x, pos, theta, inverse=False, freqs=None, mscale=1.0):
    """x [M, H, hd] float; rotate-half."""
    hd = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, hd, 2, device=x.device, dtype=torch.float32) / hd)) if freqs is None else freqs
    ang = pos.float().unsqueeze(-1) * inv
    c, s = ang.cos().unsqueeze(1) * mscale, ang.sin().unsqueeze(1) * mscale
    if inverse:
        s = -s
    x1, x2 = x[..., : hd // 2].float(), x[..., hd // 2:].float()
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)


def interleave_gate_up(gate_w: torch.Tensor, up_w: torch.Tensor, block: int = 16) -> torch.Tensor:
    """[F, d] gate and up -> [2F, d] with rows in blocks of 16: gate rows, then the matching up rows."""
    F, d = gate_w.shape
    return torch.stack([gate_w.view(F // block, block, d), up_w.view(F // block, block, d)], dim=1).reshape(2 * F, d)


def deinterleave_gate_up(gu: torch.Tensor, block: int = 16) -> tuple[torch.Tensor, torch.Tensor]:
    """Inverse of the column interleave on activations [M, 2F] -> (gate [M,F], up [M,F])."""
    M, F2 = gu.shape
    v = gu.view(M, F2 // (2 * block), 2, block)
    return v[:, :, 0].reshape(M, F2 // 2), v[:, :, 1].reshape(M, F2 // 2)
