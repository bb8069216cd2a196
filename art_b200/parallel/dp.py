"""Data parallelism for LoRA training: one process per GPU, frozen base weights replicated,
the flat fp32 LoRA gradient buffer summed across ranks before the optimizer step.

Two gradient-sync implementations:

``nccl``   ``torch.distributed.all_reduce`` on the flat buffer (the library baseline).
``fused``  the in-tree NVLink kernel (``csrc/comm/symm_mem.cu: lora_grad_allreduce_kernel``): every rank
           reduces its 1/P slice by reading the peers' symmetric buffers directly and
           writes the sum back to all peers, with bounded flag waits.

The reference has no data parallelism at all (one packed row per optimizer step on one GPU,
``src/art/local/service.py:96-118``); this module exists for the multi-GPU configurations.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def nccl_grad_sync(world: int, group=None):
    """Mean over the ranks of ``group`` (default: all ranks) with the library all-reduce of the group's backend."""
    def sync(flat_grads: torch.Tensor) -> None:
        dist.all_reduce(flat_grads, op=dist.ReduceOp.SUM, group=group)
        flat_grads.div_(world)
    return sync


def make_grad_sync(kind: str, device: torch.device, world: int):
    """Returns ``(callable(flat_grads), name)``.  ``auto`` and ``fused`` are the in-tree kernel; a failure to set it
    up (no peer access between the GPUs, ...) is an error, never a silent switch to the library path.  NCCL runs
    only when it is asked for by name."""
    if kind in ("auto", "fused"):
        from .symm_mem import fused_allreduce_sync

        return fused_allreduce_sync(device, world), "fused-p2p-allreduce"
    if kind != "nccl":
        raise ValueError(f"unknown gradient sync {kind!r} (auto, fused, nccl)")
    return nccl_grad_sync(world), "nccl-allreduce"
