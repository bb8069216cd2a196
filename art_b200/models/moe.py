"""Sparse-expert (Qwen3-MoE style) feed-forward block on the native kernels.

Per layer: a frozen softmax/top-k router, E SwiGLU experts with per-expert LoRA on
gate/up/down.  Tokens are sorted by expert into 128-row-aligned segments, the experts run as
grouped tcgen05 GEMMs (one launch for all experts, LoRA as an extra K block, SwiGLU in the
epilogue), and a gather-based combine applies the routing weights in a fixed order.  The
backward mirrors it, including the gradient that reaches the hidden state through the routing
weights.  Nothing synchronises with the host: segment sizes stay on the device.

With ``ep`` (an :class:`art_b200.parallel.ep.ExpertParallel`) the gather / combine steps become
the all-to-all dispatch / combine over NVLink and every rank holds ``E / world`` experts.

The reference supports dense models only (its README lists dense causal LMs); the autograd
oracle for this block is ``ReferenceModel.mlp`` in ``models/reference.py``.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..ops import elementwise as ew
from ..ops import moe as moe_ops
from ..ops.gemm import gemm_tn
from .config import ModelConfig
from .weights import LoraConfig, lora_key

KPAD = 64


class GroupedLoraLinear:
    """E frozen linears [N, K] stacked along rows, each with its own LoRA factors.

    ``members``: list of (module_leaf, row_index_tensor, slot) describing how HF modules map into
    the fused per-expert weight (gate/up are interleaved into one weight; down is alone).
    ``stacks[leaf]`` = ((A_param [E,r,K], A_grad), (B_param [E,n_m,r], B_grad)) views into the flat
    LoRA buffers, or None when that module carries no adapter.
    """

    def __init__(self, weights: list[torch.Tensor], members: list[tuple[str, torch.Tensor, int]], stacks: dict,
                 r: int, scale: float):
        self.E = len(weights)
        self.N, self.K = weights[0].shape
        dev = weights[0].device
        bf = torch.bfloat16
        self.W = torch.cat(weights, 0).contiguous()                                   # [E*N, K]
        self.WT = torch.cat([w.t().contiguous() for w in weights], 0).contiguous()    # [E*K, N]
        self.members = [(leaf, rows, slot) for leaf, rows, slot in members if stacks.get(leaf) is not None]
        self.stacks = stacks
        self.r, self.scale = r, scale
        self.active = len(self.members) > 0
        if self.active:
            E, N, K = self.E, self.N, self.K
            self.A_all = torch.zeros(E * KPAD, K, dtype=bf, device=dev)
            self.B_all = torch.zeros(E * N, KPAD, dtype=bf, device=dev)
            self.A_allT = torch.zeros(E * K, KPAD, dtype=bf, device=dev)
            self.B_allT = torch.zeros(E * KPAD, N, dtype=bf, device=dev)
            self.dA_acc = torch.zeros(E, K, KPAD, dtype=torch.float32, device=dev)
            self.dB_acc = torch.zeros(E, N, KPAD, dtype=torch.float32, device=dev)

    def refresh(self) -> None:
        if not self.active:
            return
        E, N, K, r = self.E, self.N, self.K, self.r
        A3 = self.A_all.view(E, KPAD, K)
        B3 = self.B_all.view(E, N, KPAD)
        for leaf, rows, slot in self.members:
            (a_p, _), (b_p, _) = self.stacks[leaf]
            c0 = slot * r
            A3[:, c0:c0 + r, :] = a_p
            B3[:, rows, c0:c0 + r] = (b_p * self.scale).to(torch.bfloat16)
        self.A_allT.view(E, K, KPAD).copy_(A3.transpose(1, 2))
        self.B_allT.view(E, KPAD, N).copy_(B3.transpose(1, 2))

    def zero_grad(self) -> None:
        if self.active:
            self.dA_acc.zero_()
            self.dB_acc.zero_()

    def export_grads(self) -> None:
        if not self.active:
            return
        r = self.r
        for leaf, rows, slot in self.members:
            (_, a_g), (_, b_g) = self.stacks[leaf]
            c0 = slot * r
            a_g.copy_(self.dA_acc[:, :, c0:c0 + r].transpose(1, 2))
            b_g.copy_(self.dB_acc[:, rows, c0:c0 + r] * self.scale)

    def forward(self, xp, plan, use_lora=True, swiglu_out=None):
        if self.active and use_lora:
            T = moe_ops.grouped_gemm(xp, self.A_all, plan, KPAD)
            y = moe_ops.grouped_gemm(xp, self.W, plan, self.N, a2=T, b2=self.B_all, swiglu_out=swiglu_out)
            return y, T
        return moe_ops.grouped_gemm(xp, self.W, plan, self.N, swiglu_out=swiglu_out), None

    def backward(self, dy, xp, T, plan):
        if self.active and T is not None:
            dT = moe_ops.grouped_gemm(dy, self.B_allT, plan, KPAD)
            moe_ops.grouped_wgrad(self.dA_acc, xp, dT, plan)
            moe_ops.grouped_wgrad(self.dB_acc, dy, T, plan)
            return moe_ops.grouped_gemm(dy, self.WT, plan, self.K, a2=dT, b2=self.A_allT)
        return moe_ops.grouped_gemm(dy, self.WT, plan, self.K)


@dataclass
class MoESaved:
    logits: torch.Tensor = None
    plan: object = None
    h2: torch.Tensor = None
    xp: torch.Tensor = None
    T_gu: torch.Tensor = None
    gu: torch.Tensor = None
    hact: torch.Tensor = None
    T_d: torch.Tensor = None
    yp: torch.Tensor = None
    eplan: object = None        # layout of the expert-side rows (== plan without expert parallelism)


def expert_lora_order(cfg: ModelConfig, keys: list[str]) -> list[str]:
    """Key order that makes every (layer, module type, A|B) block of expert adapters contiguous."""
    expert_keys = [k for k in keys if ".mlp.experts." in k]
    other = [k for k in keys if ".mlp.experts." not in k]
    present = set(expert_keys)
    ordered: list[str] = []
    for i in range(cfg.num_layers):
        for leaf in ("gate_proj", "up_proj", "down_proj"):
            for which in ("A", "B"):
                for e in range(cfg.num_experts):
                    k = lora_key(i, f"mlp.experts.{e}.{leaf}", which)
                    if k in present:
                        ordered.append(k)
    assert len(ordered) == len(expert_keys)
    return other + ordered


class MoEMLP:
    """Router + grouped experts + combine for one layer (all experts local)."""

    def __init__(self, cfg: ModelConfig, layer: int, base: dict[str, torch.Tensor], flat, lora_cfg: LoraConfig, device,
                 ep=None):
        self.cfg = cfg
        self.ep = ep
        dev, bf = device, torch.bfloat16
        p = f"model.layers.{layer}."
        E, d, F = cfg.num_experts, cfg.hidden_size, cfg.moe_intermediate_size
        self.E, self.k, self.norm = E, cfg.num_experts_per_tok, bool(cfg.norm_topk_prob)
        self.Epad = (E + 7) // 8 * 8
        wg = base[p + "mlp.gate.weight"].to(dev, bf)
        self.Wg = torch.zeros(self.Epad, d, dtype=bf, device=dev)
        self.Wg[:E] = wg
        self.WgT = self.Wg.t().contiguous()                       # [d, Epad]
        fidx = torch.arange(F, device=dev)
        gate_rows = (fidx // 16) * 32 + fidx % 16
        up_rows = gate_rows + 16

        def W(e, name):
            return base[p + f"mlp.experts.{e}.{name}.weight"].to(dev, bf)

        # with expert parallelism this rank holds (and trains) only its contiguous share of the experts
        local = range(E) if ep is None else range(ep.rank * ep.El, (ep.rank + 1) * ep.El)

        def stack(leaf):
            ka = [lora_key(layer, f"mlp.experts.{e}.{leaf}", "A") for e in local]
            if ka[0] not in flat.views:
                return None
            kb = [lora_key(layer, f"mlp.experts.{e}.{leaf}", "B") for e in local]
            return flat.stacked(ka), flat.stacked(kb)

        stacks = {leaf: stack(leaf) for leaf in ("gate_proj", "up_proj", "down_proj")}
        r, s = lora_cfg.r, lora_cfg.scale
        self.gu = GroupedLoraLinear([ew.interleave_gate_up(W(e, "gate_proj"), W(e, "up_proj")) for e in local],
                                    [("gate_proj", gate_rows, 0), ("up_proj", up_rows, 1)], stacks, r, s)
        self.down = GroupedLoraLinear([W(e, "down_proj") for e in local],
                                      [("down_proj", torch.arange(d, device=dev), 0)], stacks, r, s)
        self.F, self.d = F, d

    def linears(self):
        return (self.gu, self.down)

    def forward(self, h2: torch.Tensor, x2: torch.Tensor, use_lora: bool, save: bool):
        logits = gemm_tn(h2, self.Wg, out_dtype=torch.float32)[:, :self.E]
        plan = moe_ops.route(logits, self.k, self.norm)
        if self.ep is None:
            eplan = plan
            xp = moe_ops.gather(h2, plan)
        else:
            eplan = self.ep.exchange(plan)
            xp = self.ep.dispatch(h2, plan, eplan)
        hact = torch.empty((eplan.cap_rows, self.F), dtype=h2.dtype, device=h2.device)
        gu, T_gu = self.gu.forward(xp, eplan, use_lora, swiglu_out=hact)
        yp, T_d = self.down.forward(hact, eplan, use_lora)
        if self.ep is not None:
            yp = self.ep.combine_return(yp, plan, eplan)      # back in this rank's own sorted order
        x3, _ = moe_ops.combine(yp, plan, weighted=True, residual=x2)
        ctx = MoESaved(logits, plan, h2, xp, T_gu, gu, hact, T_d, yp, eplan) if save else None
        return x3, ctx

    def backward(self, dx: torch.Tensor, sv: MoESaved) -> torch.Tensor:
        plan, eplan = sv.plan, sv.eplan
        if self.ep is None:
            dyp = moe_ops.gather(dx, plan, weighted=True)
        else:
            dyp = self.ep.dispatch(dx, plan, eplan, weighted=True)
        _, dw = moe_ops.combine(sv.yp, plan, weighted=False, grad_for_dots=dx, want_out=False)
        dhact = self.down.backward(dyp, sv.hact, sv.T_d, eplan)
        dgu = ew.swiglu_bwd(dhact, sv.gu)
        del dhact
        dxp = self.gu.backward(dgu, sv.xp, sv.T_gu, eplan)
        del dgu
        if self.ep is not None:
            dxp = self.ep.combine_return(dxp, plan, eplan)
        dh2, _ = moe_ops.combine(dxp, plan, weighted=False)
        dlogits = moe_ops.router_bwd(sv.logits, plan, dw, self.norm, self.Epad)
        return gemm_tn(dlogits, self.WgT, residual=dh2)
