"""GRPO LoRA trainer with an explicit ``step()`` contract.

One :class:`Trainer` owns the frozen base model, the LoRA masters and the optimizer state
of one trainable model on one GPU (one rank of a data-/tensor-parallel group).  It consumes
packed tensors (``local/pack.py``) and performs optimizer steps; there is no background
training loop fed through a queue as in the reference
(``src/art/local/service.py:72-162`` + ``src/art/local/state.py:94-115``): the service calls
``train_packed`` and iterates the metrics it yields, one dict per optimizer step.

Two implementations share this interface:

``native``     the sm_100a path: :class:`models.native.NativeDecoder`, fused LM-head/GRPO
               loss kernel, flat fused AdamW.  CUDA only.
``reference``  plain PyTorch autograd over :class:`models.reference.ReferenceModel`; runs on
               CPU (oracle, tests) and on GPU (library baseline for the benchmarks).

Step semantics follow the reference: by default one packed row is one optimizer step
(``rows_per_optimizer_step=1``); the loss of a step is the mean over its rows of
``sum(pg * w * mask) / (sum(mask) + 1e-6)``; the learning rate is whatever the caller passes
for that call; gradients are clipped to ``max_grad_norm`` (0.1); AdamW betas (0.9, 0.99),
weight decay 0.1 (``src/art/dev/model.py:69-85``, ``src/art/local/train.py:34-153``).
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import Iterator

import torch

from ..models.config import ModelConfig
from ..models.reference import ReferenceModel, grpo_loss, shift_left
from ..models.weights import LoraConfig
from ..ops.optim import FlatAdamW

PACKED_KEYS = ("tokens", "group_ids", "parent_ids", "input_pos", "assistant_mask", "logprobs", "advantages", "weights")


@dataclass
class TrainHyper:
    learning_rate: float = 5e-6
    beta: float = 0.0
    epsilon: float = 0.2
    epsilon_high: float | None = None
    rows_per_optimizer_step: int = 1
    tokens_per_microbatch: int = 8192
    compat_row_positions: bool = False
    # activation recompute of the native decoder: "none" | "mlp" | "full", or "auto" = the cheapest that fits the
    # free device memory (the reference always checkpoints: use_gradient_checkpointing, src/art/dev/model.py:65)
    recompute: str = "auto"


class Trainer:
    def __init__(self, cfg: ModelConfig, base: dict[str, torch.Tensor], lora_cfg: LoraConfig,
                 lora_init: dict[str, torch.Tensor], device: str | torch.device = "cpu", impl: str | None = None,
                 betas=(0.9, 0.99), weight_decay: float = 0.1, max_grad_norm: float = 0.1, adam_eps: float = 1e-8,
                 attn_impl: str = "native", dp_group=None, grad_sync=None, ep=None, cp_group=None, tp_group=None,
                 tp_tokens: int = 8192, pp_group=None):
        self.cfg, self.lora_cfg = cfg, lora_cfg
        self.device = torch.device(device)
        self.impl = impl or ("native" if self.device.type == "cuda" else "reference")
        self.dp_group = dp_group
        self.grad_sync = grad_sync  # callable(flat_grads) -> None : data-parallel gradient all-reduce
        # expert parallelism (parallel.ep.ExpertParallel): experts sharded over the group, every rank trains on
        # its own rows; context parallelism (process group): every packed row is sharded over the group
        # tensor parallelism (process group): heads / feed-forward width sharded, activations token-sharded;
        # every micro-batch must hold exactly ``tp_tokens`` tokens
        # pipeline parallelism (process group, ranks in group order = stages): contiguous layer ranges per stage,
        # micro-batches flow through a 1F1B schedule, activations travel over NCCL point-to-point
        self.ep, self.cp_group, self.tp_group, self.pp_group = ep, cp_group, tp_group, pp_group
        self._cp_cache: dict = {}
        self._cp_sync = None
        self.tp = None
        # per-phase CUDA-event timing + NVTX ranges of every step (ARTB_PHASE_TIMING=1); read with phase_summary()
        from ..utils.profiling import PhaseTimer

        self.timer = PhaseTimer(self.device, enabled=os.environ.get("ARTB_PHASE_TIMING") == "1")
        if self.impl == "native":
            from ..models.native import NativeDecoder

            if tp_group is not None:
                import torch.distributed as dist
                from ..models.tp import TPDecoder
                from ..parallel.tp import TPContext

                P = dist.get_world_size(tp_group)
                # generous peer wait: a rank can be held up for seconds by first-touch allocations of a large micro-batch
                self.tp = TPContext(self.device, tp_group, tp_tokens // P, k_max=cfg.hidden_size, n_max=cfg.hidden_size,
                                    wait_ms=20000)
                self.model = TPDecoder(cfg, base, lora_cfg, lora_init, self.tp, self.device)
            else:
                layer_range = None
                if pp_group is not None:
                    import torch.distributed as dist
                    from ..parallel.pp import split_layers

                    layer_range = split_layers(cfg.num_layers, dist.get_world_size(pp_group))[dist.get_rank(pp_group)]
                self.model = NativeDecoder(cfg, base, lora_cfg, lora_init, self.device, attn_impl=attn_impl, ep=ep,
                                           layer_range=layer_range)
            self.flat = self.model.flat
            sum_group = cp_group if cp_group is not None else (tp_group if tp_group is not None else pp_group)
            if sum_group is not None:
                import torch.distributed as dist
                from ..parallel.symm_mem import FusedGradAllReduce

                # ranks of a context- or tensor-parallel group hold partial gradients of the SAME rows: sum them
                self._cp_sync = FusedGradAllReduce(self.device, dist.get_world_size(sum_group), sum_group, average=False,
                                                   wait_ms=20000)
                self._sum_group = sum_group
        else:
            from ..models.native import LoraFlat

            self.flat = LoraFlat(cfg, lora_cfg, lora_init, self.device)
            dt = torch.float32 if self.device.type == "cpu" else torch.bfloat16
            self.base = {k: v.to(self.device, dt) for k, v in base.items()}
            for v in self.flat.views.values():
                v.requires_grad_(True)
            self.model = ReferenceModel(cfg, self.base, self.flat.views, lora_cfg)
        self.last_recompute = "none"     # activation-recompute mode of the latest native step
        self.opt = FlatAdamW(self.flat.params.detach(), self.flat.grads, betas=betas, eps=adam_eps,
                             weight_decay=weight_decay, max_grad_norm=max_grad_norm)
        self.global_step = 0

    # ------------------------------------------------------------------ state
    def lora_state_dict(self) -> dict[str, torch.Tensor]:
        return {k: v.detach().clone() for k, v in self.flat.views.items()}

    def load_lora_state_dict(self, sd: dict[str, torch.Tensor]) -> None:
        with torch.no_grad():
            self.flat.load_state_dict(sd)
        if self.impl == "native":
            self.model.refresh_lora()

    def trainer_state(self) -> dict:
        return {"optimizer": {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in self.opt.state_dict().items()},
                "global_step": self.global_step}

    def load_trainer_state(self, st: dict) -> None:
        self.opt.load_state_dict({k: (v.to(self.device) if torch.is_tensor(v) else v) for k, v in st["optimizer"].items()})
        self.global_step = int(st.get("global_step", 0))

    # ------------------------------------------------------------------ training
    def train_packed(self, packed: dict[str, torch.Tensor], hyper: TrainHyper) -> Iterator[dict[str, float]]:
        """Yield one metrics dict per optimizer step over the rows of ``packed`` ([N,S] tensors)."""
        n_rows = packed["tokens"].shape[0]
        per = max(1, hyper.rows_per_optimizer_step)
        for start in range(0, n_rows, per):
            rows = {k: packed[k][start:start + per] for k in PACKED_KEYS}
            yield self.step(rows, hyper)

    def step(self, rows: dict[str, torch.Tensor], hyper: TrainHyper) -> dict[str, float]:
        if self.impl == "native" and self.pp_group is not None:
            m = self._step_native_pp(rows, hyper)
        elif self.impl == "native":
            m = self._step_native(rows, hyper)
        else:
            m = self._step_reference(rows, hyper)
        self.global_step += 1
        return m

    # ---- reference (autograd) ---------------------------------------------------------------
    def _step_reference(self, rows: dict[str, torch.Tensor], hyper: TrainHyper) -> dict[str, float]:
        dev = self.device
        rows = {k: v.to(dev) for k, v in rows.items()}
        R, S = rows["tokens"].shape
        self.flat.grads.zero_()
        total = {"loss": 0.0, "policy_loss": 0.0, "kl_div": 0.0}
        pos_all = None if hyper.compat_row_positions else rows["input_pos"]
        for r in range(R):  # one row at a time keeps the dense mask small
            one = {k: v[r:r + 1] for k, v in rows.items()}
            pos = None if pos_all is None else pos_all[r:r + 1]
            hidden = self.model.hidden_states(one["tokens"], one["group_ids"], one["parent_ids"], pos)
            nxt = shift_left(one["tokens"], 0)
            new_lp = self.model.logprobs(hidden, nxt)
            ref_lp = None
            if hyper.beta > 0:
                with torch.no_grad():
                    rh = self.model.hidden_states(one["tokens"], one["group_ids"], one["parent_ids"], pos, use_lora=False)
                    ref_lp = self.model.logprobs(rh, nxt)
            loss, met = grpo_loss(new_lp, one, hyper.epsilon, hyper.epsilon_high, hyper.beta, ref_lp)
            (loss / R).backward()
            total["loss"] += float(loss.detach()) / R
            total["policy_loss"] += float(met["policy_loss"]) / R
            total["kl_div"] += float(met["kl_div"]) / R
        for k, v in self.flat.views.items():
            if v.grad is not None:
                self.flat.grad_views[k].copy_(v.grad)
                v.grad = None
        return self._finish_step(total, hyper)

    # ---- native -------------------------------------------------------------------------------
    def _step_native(self, rows: dict[str, torch.Tensor], hyper: TrainHyper) -> dict[str, float]:
        from ..ops import elementwise as ew
        from ..ops import logprob_loss as lpl

        dev = self.device
        R, S = rows["tokens"].shape
        on_host = not rows["tokens"].is_cuda
        # next-token aligned per-token quantities (host side when the batch comes from the host,
        # so the trainable-token index list is known without a device sync)
        mask_s = shift_left(rows["assistant_mask"], False)
        denom = mask_s.sum(dim=1, keepdim=True).float() + 1e-6
        tok_w = shift_left(rows["weights"], 0.0) * mask_s.float() / denom / R
        sel_all = torch.nonzero(tok_w.reshape(-1) != 0, as_tuple=False).squeeze(1)  # host op if on_host
        rows_d = {k: v.to(dev, non_blocking=True) for k, v in rows.items()}
        tok_w_d = tok_w.to(dev, non_blocking=True)
        sel_all_d = sel_all.to(dev, non_blocking=True)
        self.model.zero_grad()
        accum = torch.zeros(4, dtype=torch.float32, device=dev)
        rows_per_micro = max(1, min(R, hyper.tokens_per_microbatch // S))
        eps_hi = hyper.epsilon if hyper.epsilon_high is None else hyper.epsilon_high
        sel_host = sel_all if on_host else sel_all.cpu()
        fwd_kw = {}
        if self.cp_group is None and self.tp is None:
            mode = hyper.recompute
            if mode == "auto":     # decided once per step, before any activation of the step is alive
                from ..models.native import pick_recompute

                free = torch.cuda.mem_get_info(dev)[0] + torch.cuda.memory_reserved(dev) - torch.cuda.memory_allocated(dev)
                mode = pick_recompute(self.cfg, rows_per_micro * S, len(self.model.layers), free)
            self.last_recompute = mode
            fwd_kw["recompute"] = mode
        for r0 in range(0, R, rows_per_micro):
            r1 = min(R, r0 + rows_per_micro)
            M = (r1 - r0) * S
            flat = lambda k: rows_d[k][r0:r1].reshape(-1)  # noqa: E731
            tokens = flat("tokens")
            pos = (torch.arange(S, device=dev, dtype=torch.int32).repeat(r1 - r0) if hyper.compat_row_positions
                   else flat("input_pos").to(torch.int32))
            # id compression runs where the batch lives: on the host for host batches (no device sync)
            gid, pid = compress_ids(rows["group_ids"][r0:r1].reshape(-1), rows["parent_ids"][r0:r1].reshape(-1))
            gid, pid = gid.to(dev, non_blocking=True), pid.to(dev, non_blocking=True)
            lo = int(torch.searchsorted(sel_host, r0 * S))
            hi = int(torch.searchsorted(sel_host, r1 * S))
            if hi == lo and self.cp_group is None and self.tp is None:
                continue
            target = torch.cat([tokens[1:], tokens[:1]]).to(torch.int32)  # next token; row ends are masked out
            w_flat = tok_w_d.reshape(-1)[r0 * S:r1 * S]
            old_flat = shift_left(rows_d["logprobs"][r0:r1], 0.0).reshape(-1)
            adv_flat = shift_left(rows_d["advantages"][r0:r1], 0.0).reshape(-1)
            cp = None
            if self.cp_group is not None:
                # every rank keeps its zig-zag share of each row; ids stay full-length for the mask
                cp = self._cp(r1 - r0, S)
                loc = cp.local_to_global.long()
                tokens, pos, target = tokens[loc], pos[loc].contiguous(), target[loc]
                w_flat, old_flat, adv_flat = w_flat[loc], old_flat[loc], adv_flat[loc]
                sel = torch.nonzero(w_flat != 0, as_tuple=False).squeeze(1)
            elif self.tp is not None:
                # this rank embeds, normalises and scores its contiguous token segment; positions and ids stay
                # full-length because attention runs over all tokens for the local heads
                if M != self.tp.world * self.tp.m_seg:
                    raise ValueError(f"tensor-parallel micro-batches must hold {self.tp.world * self.tp.m_seg} tokens, got {M}")
                seg = slice(self.tp.rank * self.tp.m_seg, (self.tp.rank + 1) * self.tp.m_seg)
                tokens, target = tokens[seg], target[seg]
                w_flat, old_flat, adv_flat = w_flat[seg], old_flat[seg], adv_flat[seg]
                sel = torch.nonzero(w_flat != 0, as_tuple=False).squeeze(1)
            else:
                sel = sel_all_d[lo:hi] - r0 * S
            with self.timer.phase("forward"):
                hidden, saved, final = self.model.forward(tokens, pos, gid, pid, S, cp=cp, **fwd_kw)
            if sel.numel() == 0:
                # context parallel: this rank's shard holds no trainable token, but its peers still need its
                # K/V in the forward passes and its (zero) dK/dV in the backward pass
                if hyper.beta > 0:
                    self.model.forward(tokens, pos, gid, pid, S, use_lora=False, save=False, cp=cp)
                self.model.backward(torch.zeros_like(hidden), saved, final, pos)
                continue
            hc = ew.gather_rows(hidden, sel)
            tgt_c = target[sel]
            w_c = w_flat[sel]
            old_c = old_flat[sel]
            adv_c = adv_flat[sel]
            ref_c = None
            if hyper.beta > 0:
                ref_hidden, _, _ = self.model.forward(tokens, pos, gid, pid, S, use_lora=False, save=False, cp=cp)
                rc = ew.gather_rows(ref_hidden, sel)
                part, _ = lpl.partials(rc, self.model.lm_head, tgt_c)
                ref_c = lpl.grpo_tokens(part).logprobs
                del ref_hidden, rc, part
            with self.timer.phase("lm_head_loss"):
                res = lpl.forward(hc, self.model.lm_head, tgt_c, old_c, adv_c, w_c, ref_c, hyper.epsilon, eps_hi,
                                  hyper.beta, accum)
                dhc = lpl.backward(hc, self.model.lm_head, self.model.lm_head_t, tgt_c, res.lse, res.coef)
                dhidden = torch.zeros_like(hidden)
                ew.scatter_rows_(dhc, sel, dhidden)
                del hc, dhc
            with self.timer.phase("backward"):
                self.model.backward(dhidden, saved, final, pos)
        self.model.export_grads()
        acc = accum  # read back together with the grad norm below
        out = self._finish_step(None, hyper, device_accum=acc)
        self.model.refresh_lora()
        return out

    # ---- native, pipeline parallel ---------------------------------------------------------------
    def _step_native_pp(self, rows: dict[str, torch.Tensor], hyper: TrainHyper) -> dict[str, float]:
        """One optimizer step with the layers split over the stages of ``pp_group`` (every stage sees the same rows).

        Each micro-batch is one unit of the 1F1B schedule: stage s receives the residual stream [M, d] from stage s-1,
        runs its layers, sends it on; the last stage applies the final norm, the fused LM-head loss and starts the
        backward, whose input gradient travels the other way.  Every stage accumulates the LoRA gradients of its own
        layers; the flat gradient buffers are summed over the group before the (replicated) optimizer step.
        """
        from ..ops import elementwise as ew
        from ..ops import logprob_loss as lpl
        from ..parallel.pp import PipelineRunner

        dev = self.device
        R, S = rows["tokens"].shape
        mask_s = shift_left(rows["assistant_mask"], False)
        denom = mask_s.sum(dim=1, keepdim=True).float() + 1e-6
        tok_w = (shift_left(rows["weights"], 0.0) * mask_s.float() / denom / R).to(dev)
        rows_d = {k: v.to(dev, non_blocking=True) for k, v in rows.items()}
        self.model.zero_grad()
        self.flat.grads.zero_()      # the factors of other stages' layers contribute zeros to the sum over the group
        accum = torch.zeros(4, dtype=torch.float32, device=dev)
        per = max(1, min(R, hyper.tokens_per_microbatch // S))
        if R % per:
            raise ValueError("pipeline micro-batches must all have the same number of rows")
        eps_hi = hyper.epsilon if hyper.epsilon_high is None else hyper.epsilon_high
        model, trainer = self.model, self
        micro = []
        for r0 in range(0, R, per):
            r1 = r0 + per
            tokens = rows_d["tokens"][r0:r1].reshape(-1)
            pos = (torch.arange(S, device=dev, dtype=torch.int32).repeat(per) if hyper.compat_row_positions
                   else rows_d["input_pos"][r0:r1].reshape(-1).to(torch.int32))
            gid, pid = compress_ids(rows["group_ids"][r0:r1].reshape(-1), rows["parent_ids"][r0:r1].reshape(-1))
            micro.append(dict(tokens=tokens, pos=pos, gid=gid.to(dev), pid=pid.to(dev), r0=r0, r1=r1))

        ref_lp: dict[int, torch.Tensor] = {}     # micro-batch -> reference log-probs of its trainable tokens (last stage)

        class _Stage:
            def __init__(self):
                self.live: dict = {}

            def forward(self, mb, x):
                m = micro[mb]
                with trainer.timer.phase("forward"):
                    hidden, saved, final = model.forward(m["tokens"], m["pos"], m["gid"], m["pid"], S, x_in=x)
                if not model.is_last:
                    self.live[mb] = (saved, final, None)
                    return hidden
                r0, r1 = m["r0"], m["r1"]
                w_flat = tok_w.reshape(-1)[r0 * S:r1 * S]
                sel = torch.nonzero(w_flat != 0, as_tuple=False).squeeze(1)
                dhidden = torch.zeros_like(hidden)
                if sel.numel():
                    target = torch.cat([m["tokens"][1:], m["tokens"][:1]]).to(torch.int32)
                    old_c = shift_left(rows_d["logprobs"][r0:r1], 0.0).reshape(-1)[sel]
                    adv_c = shift_left(rows_d["advantages"][r0:r1], 0.0).reshape(-1)[sel]
                    hc = ew.gather_rows(hidden, sel)
                    with trainer.timer.phase("lm_head_loss"):
                        res = lpl.forward(hc, model.lm_head, target[sel], old_c, adv_c, w_flat[sel], ref_lp.get(mb),
                                          hyper.epsilon, eps_hi, hyper.beta, accum)
                        dhc = lpl.backward(hc, model.lm_head, model.lm_head_t, target[sel], res.lse, res.coef)
                    ew.scatter_rows_(dhc, sel, dhidden)
                self.live[mb] = (saved, final, dhidden)
                return None

            def backward(self, mb, dy):
                saved, final, dhidden = self.live.pop(mb)
                with trainer.timer.phase("backward"):
                    return model.backward(dhidden if model.is_last else dy, saved, final, micro[mb]["pos"])

        runner = PipelineRunner(_Stage(), self.pp_group, act_shape=(per * S, self.cfg.hidden_size),
                                act_dtype=torch.bfloat16, device=dev)
        if hyper.beta > 0:
            # KL term: the reference policy is the frozen base model, i.e. the same stages without their LoRA factors.
            # One forward-only sweep of all micro-batches leaves the reference log-probs of the trainable tokens on
            # the last stage, where the loss of the main schedule reads them.
            def reference(mb, x):
                m = micro[mb]
                hidden, _, _ = model.forward(m["tokens"], m["pos"], m["gid"], m["pid"], S, use_lora=False, save=False, x_in=x)
                if not model.is_last:
                    return hidden
                w_flat = tok_w.reshape(-1)[m["r0"] * S:m["r1"] * S]
                sel = torch.nonzero(w_flat != 0, as_tuple=False).squeeze(1)
                if sel.numel():
                    target = torch.cat([m["tokens"][1:], m["tokens"][:1]]).to(torch.int32)
                    part, _ = lpl.partials(ew.gather_rows(hidden, sel), model.lm_head, target[sel])
                    ref_lp[mb] = lpl.grpo_tokens(part).logprobs
                return None

            runner.run_forward(len(micro), reference)
        runner.run(len(micro))
        self.model.export_grads()
        out = self._finish_step(None, hyper, device_accum=accum)
        self.model.refresh_lora()
        return out

    def _cp(self, rows: int, S: int):
        key = (rows, S)
        if key not in self._cp_cache:
            from ..parallel.cp import ContextParallel

            c = self.cfg
            self._cp_cache[key] = ContextParallel(self.device, self.cp_group, rows, S, c.num_heads, c.num_kv_heads,
                                                  c.head_dim, c.num_layers)
        return self._cp_cache[key]

    def _sync_grads(self, device_accum: torch.Tensor | None) -> None:
        """Combine the LoRA gradients of the parallel groups this trainer is part of.

        context parallel: every rank holds a partial gradient of the same rows -> sum (and the loss terms too);
        expert parallel:  non-expert factors are averaged over the group like data parallelism; an expert's
                          factors already received every rank's rows, so they are only scaled by 1/world;
        data parallel:    mean over ranks (``grad_sync``).
        """
        import torch.distributed as dist

        if self._cp_sync is not None:
            self._cp_sync(self.flat.grads)
            if device_accum is not None:
                dist.all_reduce(device_accum, group=self._sum_group)
        if self.ep is not None:
            first = [self.flat.offsets[k] for k in self.flat.names if ".mlp.experts." in k]
            n_shared = min(first) if first else self.flat.numel
            if self.grad_sync is not None:
                self.grad_sync(self.flat.grads[:n_shared])
            else:
                dist.all_reduce(self.flat.grads[:n_shared], group=self.ep.group)
                self.flat.grads[:n_shared].div_(self.ep.world)
            self.flat.grads[n_shared:].div_(self.ep.world)
        elif self.grad_sync is not None:
            self.grad_sync(self.flat.grads)
            if device_accum is not None and self.dp_group is not None:
                # loss terms are per-rank means over that rank's rows: report the mean over the data-parallel ranks
                dist.all_reduce(device_accum[:2], group=self.dp_group)
                device_accum[:2].div_(dist.get_world_size(self.dp_group))

    def phase_summary(self, group=None) -> dict[str, float]:
        """Milliseconds per phase (forward, lm_head_loss, backward, grad_sync, optimizer) since the last call."""
        return self.timer.summary(group)

    def _finish_step(self, totals: dict | None, hyper: TrainHyper, device_accum: torch.Tensor | None = None):
        with self.timer.phase("grad_sync"):
            self._sync_grads(device_accum)
        with self.timer.phase("optimizer"):
            gnorm = self.opt.step(hyper.learning_rate)
        if device_accum is not None:
            vals = torch.cat([device_accum[:2], gnorm.reshape(1)]).tolist()  # one D2H read per step
            pl, kl, gn = vals
            totals = {"policy_loss": pl, "kl_div": kl, "loss": pl + hyper.beta * kl}
        else:
            gn = float(gnorm)
            if self.dp_group is not None:      # host-side loss terms of the autograd path: mean over the data ranks
                import torch.distributed as dist

                t = torch.tensor([totals["loss"], totals["policy_loss"], totals["kl_div"]], dtype=torch.float64)
                t = t.to(self.device) if self.device.type == "cuda" else t
                dist.all_reduce(t, group=self.dp_group)
                t = (t / dist.get_world_size(self.dp_group)).tolist()
                totals = {"loss": t[0], "policy_loss": t[1], "kl_div": t[2]}
        out = {"loss": totals["loss"], "grad_norm": gn, "policy_loss": totals["policy_loss"],
               "learning_rate": hyper.learning_rate}
        if hyper.beta > 0:
            out["kl_div"] = totals["kl_div"]
        return out


def compress_ids(group_ids: torch.Tensor, parent_ids: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Map the random int64 group / parent ids of a micro-batch to dense int32 ids (order-free)."""
    both = torch.cat([group_ids, parent_ids])
    _, inv = torch.unique(both, return_inverse=True)
    n = group_ids.numel()
    return inv[:n].to(torch.int32).contiguous(), inv[n:].to(torch.int32).contiguous()
