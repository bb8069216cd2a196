"""Flat-buffer AdamW with device-side global-norm clipping (``csrc/kernels/adamw.cu``)."""
from __future__ import annotations

import ctypes

import torch

from . import _lib

vp, ci, cf, cl = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_long
_bound: dict[str, object] = {}
_sigs = {
    "artb_grad_sumsq": [vp, cl, cf, vp, vp],
    "artb_adamw_step": [vp, vp, vp, vp, cl, cf, cf, cf, cf, cf, ci, cf, cf, vp, vp],
}


def _f(name: str):
    fn = _bound.get(name)
    if fn is None:
        fn = getattr(_lib.kernels(), name)
        fn.argtypes = _sigs[name]
        fn.restype = ci
        _bound[name] = fn
    return fn


class FlatAdamW:
    """AdamW over one contiguous fp32 parameter buffer.

    ``params`` / ``grads`` are 1-D fp32 tensors of equal length; per-parameter tensors are
    views into them.  On CUDA the fused kernels run; on CPU the same arithmetic runs in
    PyTorch (used by the CPU tests and the oracle comparison).
    """

    def __init__(self, params: torch.Tensor, grads: torch.Tensor, betas=(0.9, 0.99), eps: float = 1e-8,
                 weight_decay: float = 0.1, max_grad_norm: float = 0.1):
        assert params.dim() == 1 and params.dtype == torch.float32 and params.shape == grads.shape
        self.params, self.grads = params, grads
        self.m = torch.zeros_like(params)
        self.v = torch.zeros_like(params)
        self.betas, self.eps, self.weight_decay, self.max_grad_norm = betas, eps, weight_decay, max_grad_norm
        self.step_count = 0
        self.stats = torch.zeros(4, dtype=torch.float32, device=params.device)

    def step(self, lr: float, grad_scale: float = 1.0) -> torch.Tensor:
        """Apply one update; returns a 0-d tensor with the pre-clip gradient norm."""
        self.step_count += 1
        b1, b2 = self.betas
        n = self.params.numel()
        if self.params.is_cuda:
            self.stats.zero_()
            _lib.check_rc(_f("artb_grad_sumsq")(_lib.ptr(self.grads), n, grad_scale, _lib.ptr(self.stats),
                                                _lib.stream_ptr()), "grad_sumsq")
            _lib.check_rc(_f("artb_adamw_step")(_lib.ptr(self.params), _lib.ptr(self.grads), _lib.ptr(self.m),
                                                _lib.ptr(self.v), n, lr, b1, b2, self.eps, self.weight_decay,
                                                self.step_count, self.max_grad_norm, grad_scale,
                                                _lib.ptr(self.stats), _lib.stream_ptr()), "adamw_step")
            return self.stats[1]
        g = self.grads * grad_scale
        norm = g.norm()
        if self.max_grad_norm > 0:
            g = g * torch.clamp(self.max_grad_norm / (norm + 1e-6), max=1.0)
        self.params.mul_(1 - lr * self.weight_decay)
        self.m.mul_(b1).add_(g, alpha=1 - b1)
        self.v.mul_(b2).addcmul_(g, g, value=1 - b2)
        bias1, bias2 = 1 - b1 ** self.step_count, 1 - b2 ** self.step_count
        denom = (self.v.sqrt() / (bias2 ** 0.5)).add_(self.eps)
        self.params.addcdiv_(self.m, denom, value=-lr / bias1)
        return norm

    def state_dict(self) -> dict:
        return {"m": self.m, "v": self.v, "step": self.step_count}

    def load_state_dict(self, sd: dict) -> None:
        self.m.copy_(sd["m"])
        self.v.copy_(sd["v"])
        self.step_count = int(sd["step"])
