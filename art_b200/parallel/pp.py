"""Pipeline parallelism: 1F1B schedule with NCCL (or gloo) point-to-point activation transfer.

Stage ``s`` of ``P`` runs ``min(P - s - 1, n_micro)`` warm-up forwards, then alternates one forward
and one backward, then drains the remaining backwards.  Activations travel downstream and
activation gradients upstream as grouped ``isend`` / ``irecv`` pairs; on CUDA they run on the
transport's own stream, so a send overlaps the next micro-batch's compute.

A stage is any object with

    forward(mb: int, x: Tensor | None) -> Tensor      (first stage gets None; last stage returns
                                                        anything, e.g. the loss, and sends nothing)
    backward(mb: int, dy: Tensor | None) -> Tensor | None   (last stage gets None; first stage's
                                                        return value is ignored)

The reference has no pipeline parallelism of its own (``pipeline_parallel_size`` is forwarded to
the inference library, ``src/art/dev/engine.py:26``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Protocol

import torch
import torch.distributed as dist


def schedule_1f1b(stage: int, n_stages: int, n_micro: int) -> list[tuple[str, int]]:
    """Operation order of one stage: a list of ("F", micro_batch) / ("B", micro_batch)."""
    if not (0 <= stage < n_stages) or n_micro < 1:
        raise ValueError("bad pipeline geometry")
    warm = min(n_stages - stage - 1, n_micro)
    ops: list[tuple[str, int]] = [("F", i) for i in range(warm)]
    f, b = warm, 0
    while f < n_micro:
        ops.append(("F", f))
        f += 1
        ops.append(("B", b))
        b += 1
    while b < n_micro:
        ops.append(("B", b))
        b += 1
    return ops


def peak_in_flight(stage: int, n_stages: int, n_micro: int) -> int:
    """Largest number of micro-batches whose activations a stage holds at once under 1F1B."""
    live = peak = 0
    for kind, _ in schedule_1f1b(stage, n_stages, n_micro):
        live += 1 if kind == "F" else -1
        peak = max(peak, live)
    return peak


class Stage(Protocol):
    def forward(self, mb: int, x: torch.Tensor | None) -> Any: ...

    def backward(self, mb: int, dy: torch.Tensor | None) -> torch.Tensor | None: ...


class _Once:
    """A transfer handle that is waited on at most once (a second wait on a finished gloo send blocks)."""

    def __init__(self, work):
        self.work = work

    def wait(self) -> None:
        w, self.work = self.work, None
        if w is not None:
            w.wait()


@dataclass
class _Pending:
    works: list
    tensor: torch.Tensor | None


class PipelineRunner:
    """Drives one stage of a 1F1B pipeline over a process group (ranks in group order = stages).

    After each compute operation the stage issues, as ONE grouped point-to-point call per peer,
    the send of what it just produced and the receive of what its next operation consumes
    (send-forward/receive-backward and send-backward/receive-forward in the steady state, which
    target the same neighbour and therefore cannot dead-lock on in-order transports).  The calls
    are asynchronous: the transport's own stream carries them while the compute stream goes on,
    and the stage only waits for a receive right before the operation that needs it.
    """

    def __init__(self, stage: Stage, group=None, act_shape: tuple[int, ...] = (), act_dtype=torch.bfloat16,
                 device: torch.device | str = "cpu"):
        self.stage_obj = stage
        self.group = group
        self.stage = dist.get_rank(group)
        self.n_stages = dist.get_world_size(group)
        self.act_shape, self.act_dtype = tuple(act_shape), act_dtype
        self.device = torch.device(device)
        self.bytes_sent = 0

    def _peer(self, delta: int) -> int:
        r = self.stage + delta
        return dist.get_global_rank(self.group, r) if self.group is not None else r

    def _exchange(self, send_t: torch.Tensor | None, send_delta: int, recv_delta: int | None):
        """Returns (send_pending | None, recv_pending | None)."""
        send_op = recv_op = None
        buf = None
        if send_t is not None:
            send_t = send_t.contiguous()
            self.bytes_sent += send_t.numel() * send_t.element_size()
            send_op = dist.P2POp(dist.isend, send_t, self._peer(send_delta), self.group)
        if recv_delta is not None:
            buf = torch.empty(self.act_shape, dtype=self.act_dtype, device=self.device)
            recv_op = dist.P2POp(dist.irecv, buf, self._peer(recv_delta), self.group)
        if send_op is not None and recv_op is not None and send_delta == recv_delta:
            works = [_Once(w) for w in dist.batch_isend_irecv([send_op, recv_op])]
            return _Pending(works, send_t), _Pending(works, buf)
        sp = rp = None
        if send_op is not None:
            sp = _Pending([_Once(w) for w in dist.batch_isend_irecv([send_op])], send_t)
        if recv_op is not None:
            rp = _Pending([_Once(w) for w in dist.batch_isend_irecv([recv_op])], buf)
        return sp, rp

    # -- schedule -------------------------------------------------------------------------------
    def run(self, n_micro: int) -> list[Any]:
        """Execute one optimizer step's worth of micro-batches; returns the last stage's forward outputs."""
        return self._run(schedule_1f1b(self.stage, self.n_stages, n_micro), self.stage_obj.forward, self.stage_obj.backward)

    def run_forward(self, n_micro: int, fn) -> list[Any]:
        """A forward-only sweep of all micro-batches through the stages, in order (no activations are kept, so nothing
        limits how many are in flight): ``fn(mb, x)`` returns the tensor to send downstream; on the last stage its
        return values are collected.  Used for the reference-policy pass of the KL term."""
        return self._run([("F", i) for i in range(n_micro)], fn, None)

    def _run(self, ops: list[tuple[str, int]], fwd, bwd) -> list[Any]:
        first, last = self.stage == 0, self.stage == self.n_stages - 1
        sends: list[_Pending] = []
        outputs: list[Any] = []

        def recv_delta(op):
            kind, _ = op
            if kind == "F":
                return None if first else -1
            return None if last else +1

        _, pending = self._exchange(None, 0, recv_delta(ops[0]))
        for i, op in enumerate(ops):
            kind, mb = op
            inp = None
            if pending is not None:
                for w in pending.works:
                    w.wait()
                inp = pending.tensor
            send_t, send_delta = None, 0
            if kind == "F":
                out = fwd(mb, inp)
                if last:
                    outputs.append(out)
                else:
                    send_t, send_delta = out, +1
            else:
                dx = bwd(mb, inp)
                if not first:
                    send_t, send_delta = dx, -1
            nxt = recv_delta(ops[i + 1]) if i + 1 < len(ops) else None
            sp, pending = self._exchange(send_t, send_delta, nxt)
            if sp is not None:
                sends.append(sp)
        for p in sends:
            for w in p.works:
                w.wait()
        return outputs


def split_layers(n_layers: int, n_stages: int) -> list[range]:
    """Contiguous, near-equal layer ranges; earlier stages take the remainder."""
    base, rem = divmod(n_layers, n_stages)
    out, lo = [], 0
    for s in range(n_stages):
        hi = lo + base + (1 if s < rem else 0)
        out.append(range(lo, hi))
        lo = hi
    return out
