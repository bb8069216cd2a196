"""Fused LM-head log-prob + GRPO loss (``csrc/kernels/logprob_loss.cu``).

``forward`` returns per-token log-probs and accumulates the loss terms without ever
materialising logits; ``backward`` recomputes logit tiles, writes bf16 ``dlogits`` and
contracts them with the resident transposed LM head on the tcgen05 GEMM.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _lib
from .gemm import gemm_tn

vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
_bound: dict[str, object] = {}
_sigs = {
    "artb_logprob_splits": [ci, ci],
    "artb_logprob_partials": [vp, ci, vp, ci, vp, vp, ci, ci, ci, ci, ci, vp, vp],
    "artb_grpo_tokens": [vp, ci, ci, vp, vp, vp, vp, cf, cf, cf, vp, vp, vp, vp, vp],
    "artb_logprob_dlogits": [vp, ci, vp, ci, vp, vp, vp, vp, ci, ci, ci, ci, ci, vp, vp],
}


def _f(name: str):
    fn = _bound.get(name)
    if fn is None:
        fn = getattr(_lib.kernels(), name)
        fn.argtypes = _sigs[name]
        fn.restype = ci
        _bound[name] = fn
    return fn


@dataclass
class LogprobResult:
    logprobs: torch.Tensor      # [M] fp32
    lse: torch.Tensor           # [M] fp32
    coef: torch.Tensor | None   # [M] dLoss/dlogprob (None for a stats-only pass)
    accum: torch.Tensor | None  # [4] fp32: sum(pg*w), sum(kl*w), #tokens with w != 0


def partials(hidden: torch.Tensor, lm_head: torch.Tensor, target: torch.Tensor, vocab_offset: int = 0
             ) -> tuple[torch.Tensor, int]:
    """Per-vocab-split (max, sumexp, z_target) for one vocabulary shard: [splits, M, 4] fp32."""
    M, K = hidden.shape
    V = lm_head.shape[0]
    splits = _f("artb_logprob_splits")(M, V)
    part = torch.empty((splits, M, 4), dtype=torch.float32, device=hidden.device)
    rc = _f("artb_logprob_partials")(_lib.ptr(hidden), hidden.stride(0), _lib.ptr(lm_head), lm_head.stride(0),
                                     _lib.ptr(target), _lib.ptr(part), M, V, K, splits, vocab_offset,
                                     _lib.ptr(_lib.status_word(hidden.device)), _lib.stream_ptr())
    _lib.check_rc(rc, "logprob_partials")
    return part, splits


def grpo_tokens(part: torch.Tensor, old_lp=None, adv=None, tok_w=None, ref_lp=None, eps_lo: float = 0.2,
                eps_hi: float = 0.2, beta: float = 0.0, accum: torch.Tensor | None = None) -> LogprobResult:
    splits, M, _ = part.shape
    dev = part.device
    lse = torch.empty(M, dtype=torch.float32, device=dev)
    lp = torch.empty(M, dtype=torch.float32, device=dev)
    coef = torch.empty(M, dtype=torch.float32, device=dev) if tok_w is not None else None
    if tok_w is not None and accum is None:
        accum = torch.zeros(4, dtype=torch.float32, device=dev)
    rc = _f("artb_grpo_tokens")(_lib.ptr(part), splits, M, _lib.ptr(old_lp), _lib.ptr(adv), _lib.ptr(tok_w),
                                _lib.ptr(ref_lp), eps_lo, eps_hi, beta, _lib.ptr(lse), _lib.ptr(lp), _lib.ptr(coef),
                                _lib.ptr(accum), _lib.stream_ptr())
    _lib.check_rc(rc, "grpo_tokens")
    return LogprobResult(lp, lse, coef, accum)


def forward(hidden, lm_head, target, old_lp=None, adv=None, tok_w=None, ref_lp=None, eps_lo=0.2, eps_hi=0.2,
            beta=0.0, accum=None) -> LogprobResult:
    """hidden [M,K] bf16, lm_head [V,K] bf16, target [M] int32 (next-token ids)."""
    part, _ = partials(hidden, lm_head, target)
    return grpo_tokens(part, old_lp, adv, tok_w, ref_lp, eps_lo, eps_hi, beta, accum)


def backward(hidden, lm_head, lm_head_t, target, lse, coef, dlogits_buf: torch.Tensor | None = None) -> torch.Tensor:
    """dH [M,K] bf16.  ``lm_head_t`` is the resident [K, ldo] transposed head (ldo = V padded to 8)."""
    M, K = hidden.shape
    V = lm_head.shape[0]
    ldo = lm_head_t.shape[1]
    if dlogits_buf is None or dlogits_buf.shape[0] < M:
        dlogits_buf = torch.empty((M, ldo), dtype=torch.bfloat16, device=hidden.device)
    dl = dlogits_buf[:M]
    rc = _f("artb_logprob_dlogits")(_lib.ptr(hidden), hidden.stride(0), _lib.ptr(lm_head), lm_head.stride(0),
                                    _lib.ptr(target), _lib.ptr(lse), _lib.ptr(coef), _lib.ptr(dl), ldo, M, V, K, 0,
                                    _lib.ptr(_lib.status_word(hidden.device)), _lib.stream_ptr())
    _lib.check_rc(rc, "logprob_dlogits")
    return gemm_tn(dl, lm_head_t)


def reference_logprobs(hidden, lm_head, target):
    logits = hidden.float() @ lm_head.float().t()
    return logits.gather(-1, target.long().unsqueeze(-1)).squeeze(-1) - torch.logsumexp(logits, -1)
