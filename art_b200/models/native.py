"""Dense decoder with hand-scheduled forward and backward on the sm_100a kernels.

There is no autograd graph: the layer structure is fixed, base weights are frozen, and
only LoRA factors receive gradients, so forward and backward are two explicit sequences
of kernel launches over preallocated activations.  Design points:

* Every projection is ONE tcgen05 GEMM.  q/k/v are fused into one weight, gate/up into
  one (row-interleaved in blocks of 16 so the SwiGLU sits in the GEMM epilogue).  The LoRA
  update rides along as an extra 64-wide K block: ``T = X @ A_cat.T`` (a skinny GEMM) and
  then ``Y = [X | T] @ [W | s*B_cat].T`` accumulate in the same TMEM tile.
* The data gradient uses a resident transposed copy of each frozen weight, so it is a
  K-major "TN" GEMM too: ``dX = [dY | dT] @ [W.T | A_cat.T].T`` with ``dT = dY @ (s*B_cat)``.
  Holding W and W.T doubles weight memory (2 x 15 GB for a 7B model), which 180 GB of HBM
  makes the right trade.
* All activations a backward pass needs are kept while a micro-batch fits.  ``recompute="mlp"``
  drops the feed-forward intermediates (gate|up pre-activations and the activation, three
  quarters of the saved bytes) and re-runs the gate|up GEMM in the backward pass;
  ``recompute="full"`` keeps only each layer's input and re-runs the whole layer forward
  (:func:`activation_bytes_per_token`, :func:`pick_recompute`).  This is what lets one GPU train
  the reference's default 32 768-token rows (``src/art/dev/model.py:28``, gradient
  checkpointing at ``:65``).
* LoRA masters/gradients live in flat fp32 buffers (:class:`LoraFlat`); the bf16 operand
  copies (A_cat, B_cat and their transposes) are rebuilt after each optimizer step.

Parity: this is the trainer-side model the reference obtains from Unsloth/PEFT
(``src/art/local/state.py:77-92``) and drives at ``src/art/local/train.py:218-242``.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..ops import attention as attn_ops
from ..ops import elementwise as ew
from ..ops.gemm import gemm_tn, skinny_gemm
from .config import ModelConfig
from .weights import LoraConfig, lora_key

LORA_KPAD = 64  # extra-K block width


@dataclass
class _Member:
    module: str            # e.g. "self_attn.q_proj"
    rows: torch.Tensor     # int64 row indices of this member inside the fused weight
    slot: int              # member uses T columns [slot*r, (slot+1)*r)
    a_view: torch.Tensor = None   # fp32 views into the flat master / grad buffers
    b_view: torch.Tensor = None
    ga_view: torch.Tensor = None
    gb_view: torch.Tensor = None


class LoraLinear:
    """A fused frozen linear (one or several HF modules) with per-member LoRA factors."""

    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None, members: list[_Member], r: int, scale: float,
                 need_dgrad: bool = True):
        self.W = weight.contiguous()                      # [N, K] bf16
        self.WT = weight.t().contiguous() if need_dgrad else None   # [K, N] bf16
        self.bias = bias.float().contiguous() if bias is not None else None
        self.members = members
        self.r, self.scale = r, scale
        N, K = self.W.shape
        dev = self.W.device
        self.active = len(members) > 0
        self.kpad = max(LORA_KPAD, ((len(members) * r + 63) // 64) * 64)
        if self.active:
            self.A_cat = torch.zeros(self.kpad, K, dtype=torch.bfloat16, device=dev)
            self.B_cat = torch.zeros(N, self.kpad, dtype=torch.bfloat16, device=dev)
            self.A_catT = torch.zeros(K, self.kpad, dtype=torch.bfloat16, device=dev)
            self.B_catT = torch.zeros(self.kpad, N, dtype=torch.bfloat16, device=dev)
            self.dA_acc = torch.zeros(K, self.kpad, dtype=torch.float32, device=dev)   # stored transposed: [K, kpad]
            self.dB_acc = torch.zeros(N, self.kpad, dtype=torch.float32, device=dev)

    def refresh(self) -> None:
        """Rebuild the bf16 operand copies from the fp32 masters."""
        if not self.active:
            return
        r = self.r
        for m in self.members:
            c0 = m.slot * r
            self.A_cat[c0:c0 + r] = m.a_view
            self.B_cat[m.rows, c0:c0 + r] = (m.b_view * self.scale).to(torch.bfloat16)
        self.A_catT.copy_(self.A_cat.t())
        self.B_catT.copy_(self.B_cat.t())

    def zero_grad(self) -> None:
        if self.active:
            self.dA_acc.zero_()
            self.dB_acc.zero_()

    def export_grads(self) -> None:
        """Scatter the accumulated fused gradients into the flat per-member gradient views."""
        if not self.active:
            return
        r = self.r
        for m in self.members:
            c0 = m.slot * r
            m.ga_view.copy_(self.dA_acc[:, c0:c0 + r].t())
            m.gb_view.copy_(self.dB_acc[m.rows, c0:c0 + r] * self.scale)

    # forward: returns (y, T) ; T is saved for the B-gradient
    def forward(self, x: torch.Tensor, use_lora: bool = True, residual=None, swiglu_out=None, out=None):
        if self.active and use_lora:
            T = skinny_gemm(x, self.A_cat)
            y = gemm_tn(x, self.W, a2=T, b2=self.B_cat, residual=residual, swiglu_out=swiglu_out, bias=self.bias, out=out)
            return y, T
        y = gemm_tn(x, self.W, residual=residual, swiglu_out=swiglu_out, bias=self.bias, out=out)
        return y, None

    # backward: dx, and accumulates dA_cat / dB_cat
    def backward(self, dy: torch.Tensor, x: torch.Tensor, T: torch.Tensor | None, need_dx: bool = True,
                 dx_residual: torch.Tensor | None = None, swiglu_gu: torch.Tensor | None = None) -> torch.Tensor | None:
        """``swiglu_gu``: this linear's input was ``silu(gate) * up``; return d(gate|up) instead of d(input)."""
        if self.active and T is not None:
            dT = skinny_gemm(dy, self.B_catT)                   # [M, kpad]
            # LoRA factor gradients: skinny contractions over the token dimension
            lora_wgrad(self.dA_acc, x, dT)     # dA_cat^T [K, kpad] += X^T dT
            lora_wgrad(self.dB_acc, dy, T)     # dB_cat   [N, kpad] += dY^T T
            if need_dx:
                return gemm_tn(dy, self.WT, a2=dT, b2=self.A_catT, residual=dx_residual, swiglu_bwd_gu=swiglu_gu)
            return None
        if need_dx:
            return gemm_tn(dy, self.WT, residual=dx_residual, swiglu_bwd_gu=swiglu_gu)
        return None


def lora_wgrad(acc: torch.Tensor, p: torch.Tensor, q: torch.Tensor, transpose_out: bool = False) -> None:
    """``acc += p.T @ q`` (or its transpose) for tall-skinny bf16 operands, fp32 accumulation."""
    from ..ops import wgrad

    wgrad.accumulate(acc, p, q, transpose_out)


class LoraFlat:
    """Flat fp32 master / gradient buffers holding every LoRA A and B (PEFT-named views)."""

    def __init__(self, cfg: ModelConfig, lcfg: LoraConfig, init: dict[str, torch.Tensor], device,
                 order: list[str] | None = None):
        if order is not None:
            assert sorted(order) == sorted(init.keys())
            init = {k: init[k] for k in order}
        self.names = list(init.keys())
        total = sum(v.numel() for v in init.values())
        pad = (-total) % 1024
        self.params = torch.zeros(total + pad, dtype=torch.float32, device=device)
        self.grads = torch.zeros_like(self.params)
        self.views: dict[str, torch.Tensor] = {}
        self.grad_views: dict[str, torch.Tensor] = {}
        self.offsets: dict[str, int] = {}
        off = 0
        for k, v in init.items():
            n = v.numel()
            self.views[k] = self.params[off:off + n].view(v.shape)
            self.grad_views[k] = self.grads[off:off + n].view(v.shape)
            self.views[k].copy_(v)
            self.offsets[k] = off
            off += n
        self.numel = total

    def stacked(self, keys: list[str]) -> tuple[torch.Tensor, torch.Tensor]:
        """Parameter and gradient views ``[len(keys), *shape]`` over keys that are adjacent in the flat buffer."""
        shape = self.views[keys[0]].shape
        n = self.views[keys[0]].numel()
        o0 = self.offsets[keys[0]]
        for i, k in enumerate(keys):
            if self.offsets[k] != o0 + i * n or self.views[k].shape != shape:
                raise ValueError("keys are not adjacent in the flat LoRA buffer")
        span = slice(o0, o0 + n * len(keys))
        return self.params[span].view(len(keys), *shape), self.grads[span].view(len(keys), *shape)

    def state_dict(self) -> dict[str, torch.Tensor]:
        return {k: v.detach().clone() for k, v in self.views.items()}

    def load_state_dict(self, sd: dict[str, torch.Tensor]) -> None:
        for k, v in sd.items():
            if k in self.views:
                self.views[k].copy_(v)


RECOMPUTE_MODES = ("none", "mlp", "full")


def activation_bytes_per_token(cfg: ModelConfig, mode: str = "none") -> int:
    """bf16 bytes one token keeps alive per decoder layer between forward and backward."""
    d, q, kv = cfg.hidden_size, cfg.q_size, cfg.kv_size
    F = cfg.moe_intermediate_size * cfg.num_experts_per_tok if cfg.is_moe else cfg.intermediate_size
    if mode == "full":
        return 2 * d
    attn = 4 * d + 2 * q + 2 * kv                    # x, h1, x2, h2, qkv, o
    return 2 * (attn + (0 if mode == "mlp" else 3 * F))


def pick_recompute(cfg: ModelConfig, tokens: int, num_layers: int, free_bytes: int) -> str:
    """The cheapest mode whose saved activations (plus the working set of one layer's backward pass and the LM-head
    buffers) fit into ``free_bytes``."""
    work = tokens * (4 * activation_bytes_per_token(cfg, "none") + 16 * cfg.hidden_size)
    for mode in RECOMPUTE_MODES:
        if tokens * num_layers * activation_bytes_per_token(cfg, mode) + work <= 0.85 * free_bytes:
            return mode
    return "full"


@dataclass
class LayerSaved:
    recompute: str = "none"     # what has to be rebuilt from x (full) or x2 (mlp) before this layer's backward
    x: torch.Tensor = None
    rstd1: torch.Tensor = None
    h1: torch.Tensor = None
    T_qkv: torch.Tensor = None
    attn_ctx: object = None
    o: torch.Tensor = None
    T_o: torch.Tensor = None
    x2: torch.Tensor = None
    rstd2: torch.Tensor = None
    mlp: object = None          # DenseSaved or MoESaved
    qk_pre: torch.Tensor = None
    qk_rstd: tuple = None


@dataclass
class DenseSaved:
    h2: torch.Tensor = None
    T_gu: torch.Tensor = None
    gu: torch.Tensor = None
    hact: torch.Tensor = None
    T_d: torch.Tensor = None


class DenseMLP:
    """SwiGLU feed-forward: fused gate|up GEMM with the activation in its epilogue, then down + residual."""

    def __init__(self, gu: LoraLinear, down: LoraLinear, intermediate: int):
        self.gu, self.down, self.F = gu, down, intermediate

    def linears(self):
        return (self.gu, self.down)

    def forward(self, h2, x2, use_lora: bool, save: bool):
        hact = torch.empty((h2.shape[0], self.F), dtype=h2.dtype, device=h2.device)
        gu, T_gu = self.gu.forward(h2, use_lora, swiglu_out=hact)
        x3, T_d = self.down.forward(hact, use_lora, residual=x2)
        return x3, (DenseSaved(h2, T_gu, gu, hact, T_d) if save else None)

    def recompute(self, h2, x2, use_lora: bool) -> DenseSaved:
        """What :meth:`forward` would have saved, without the down projection (its output is not needed again)."""
        hact = torch.empty((h2.shape[0], self.F), dtype=h2.dtype, device=h2.device)
        gu, T_gu = self.gu.forward(h2, use_lora, swiglu_out=hact)
        T_d = skinny_gemm(hact, self.down.A_cat) if (self.down.active and use_lora) else None
        return DenseSaved(h2, T_gu, gu, hact, T_d)

    def backward(self, dx, sv: DenseSaved):
        # the SwiGLU backward sits in the epilogue of the down-projection's data-gradient GEMM
        dgu = self.down.backward(dx, sv.hact, sv.T_d, swiglu_gu=sv.gu)
        return self.gu.backward(dgu, sv.h2, sv.T_gu)


class NativeDecoder:
    """Qwen2/Llama-style dense and Qwen3-MoE-style sparse decoders on the native kernels (LoRA-only training)."""

    def __init__(self, cfg: ModelConfig, base: dict[str, torch.Tensor], lora_cfg: LoraConfig,
                 lora_init: dict[str, torch.Tensor], device="cuda", attn_impl: str = "native", ep=None,
                 layer_range: range | None = None):
        self.cfg, self.lora_cfg, self.attn_impl = cfg, lora_cfg, attn_impl
        self.device = torch.device(device)
        ew.rope_args(cfg, self.device)       # builds the frequency table of a scaled rotary embedding now, not mid-step
        # pipeline parallelism: this instance holds the decoder layers of `layer_range` only; the first stage embeds,
        # the last applies the final norm (the LM head / loss stay with the caller, as without pipelining)
        self.layer_ids = list(layer_range) if layer_range is not None else list(range(cfg.num_layers))
        self.is_first = self.layer_ids[0] == 0
        self.is_last = self.layer_ids[-1] == cfg.num_layers - 1
        bf = torch.bfloat16
        dev = self.device
        self.embed = base["model.embed_tokens.weight"].to(dev, bf).contiguous()
        self.lm_head = base["lm_head.weight"].to(dev, bf).contiguous()
        V, d = self.lm_head.shape
        ldo = (V + 7) // 8 * 8
        self.lm_head_t = torch.zeros(d, ldo, dtype=bf, device=dev)
        self.lm_head_t[:, :V] = self.lm_head.t()
        self.final_norm = base["model.norm.weight"].to(dev, bf).contiguous()
        order = None
        if cfg.is_moe:
            from .moe import MoEMLP, expert_lora_order

            order = expert_lora_order(cfg, list(lora_init.keys()))
        self.flat = LoraFlat(cfg, lora_cfg, lora_init, dev, order=order)
        self.layers: list[dict] = []
        r, s = lora_cfg.r, lora_cfg.scale
        F = max(cfg.intermediate_size, 16)
        fidx = torch.arange(F, device=dev)
        gate_rows = (fidx // 16) * 32 + fidx % 16
        up_rows = gate_rows + 16
        for i in self.layer_ids:
            p = f"model.layers.{i}."

            def W(name):
                return base[p + name + ".weight"].to(dev, bf)

            def members(specs):
                out = []
                for slot, (module, rows) in enumerate(specs):
                    ka = lora_key(i, module, "A")
                    if ka in self.flat.views:
                        kb = lora_key(i, module, "B")
                        out.append(_Member(module, rows, slot, self.flat.views[ka], self.flat.views[kb],
                                           self.flat.grad_views[ka], self.flat.grad_views[kb]))
                return out

            q, kv = cfg.q_size, cfg.kv_size
            wqkv = torch.cat([W("self_attn.q_proj"), W("self_attn.k_proj"), W("self_attn.v_proj")], 0)
            bqkv = None
            if cfg.qkv_bias:
                bqkv = torch.cat([base[p + f"self_attn.{n}.bias"].to(dev) for n in ("q_proj", "k_proj", "v_proj")])
            ar = torch.arange
            qkv = LoraLinear(wqkv, bqkv, members([("self_attn.q_proj", ar(0, q, device=dev)),
                                                  ("self_attn.k_proj", ar(q, q + kv, device=dev)),
                                                  ("self_attn.v_proj", ar(q + kv, q + 2 * kv, device=dev))]), r, s)
            o = LoraLinear(W("self_attn.o_proj"), None, members([("self_attn.o_proj", ar(0, d, device=dev))]), r, s)
            if cfg.is_moe:
                mlp = MoEMLP(cfg, i, base, self.flat, lora_cfg, dev, ep=ep)
            else:
                wgu = ew.interleave_gate_up(W("mlp.gate_proj"), W("mlp.up_proj"))
                gu = LoraLinear(wgu, None, members([("mlp.gate_proj", gate_rows), ("mlp.up_proj", up_rows)]), r, s)
                down = LoraLinear(W("mlp.down_proj"), None, members([("mlp.down_proj", ar(0, d, device=dev))]), r, s)
                mlp = DenseMLP(gu, down, cfg.intermediate_size)
            layer = {"qkv": qkv, "o": o, "mlp": mlp,
                     "ln1": base[p + "input_layernorm.weight"].to(dev, bf).contiguous(),
                     "ln2": base[p + "post_attention_layernorm.weight"].to(dev, bf).contiguous()}
            if cfg.qk_norm:
                layer["q_norm"] = base[p + "self_attn.q_norm.weight"].to(dev, bf).contiguous()
                layer["k_norm"] = base[p + "self_attn.k_norm.weight"].to(dev, bf).contiguous()
            self.layers.append(layer)
        self.refresh_lora()

    # -- LoRA bookkeeping -------------------------------------------------------------------
    def linears(self):
        for layer in self.layers:
            yield layer["qkv"]
            yield layer["o"]
            yield from layer["mlp"].linears()

    def refresh_lora(self) -> None:
        for lin in self.linears():
            lin.refresh()

    def zero_grad(self) -> None:
        for lin in self.linears():
            lin.zero_grad()

    def export_grads(self) -> None:
        for lin in self.linears():
            lin.export_grads()

    # -- forward ----------------------------------------------------------------------------
    def _layer_forward(self, li: int, x, pos, plan, use_lora: bool, save: bool, cp=None, need_out: bool = True):
        """One decoder layer; returns (output or None, LayerSaved or None)."""
        cfg, layer = self.cfg, self.layers[li]
        Hq, Hkv, hd = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        sv = LayerSaved()
        h1, rstd1 = ew.rmsnorm_fwd(x, layer["ln1"], cfg.rms_norm_eps)
        qkv, T_qkv = layer["qkv"].forward(h1, use_lora)
        if cfg.qk_norm:
            if save:
                sv.qk_pre = qkv[:, : (Hq + Hkv) * hd].clone()
            rq = ew.headnorm_fwd_(qkv, layer["q_norm"], 0, Hq, hd, cfg.rms_norm_eps)
            rk = ew.headnorm_fwd_(qkv, layer["k_norm"], Hq * hd, Hkv, hd, cfg.rms_norm_eps)
            sv.qk_rstd = (rq, rk)
        ew.rope_(qkv, pos, 0, Hq + Hkv, hd, cfg.rope_theta, **ew.rope_args(cfg, qkv.device))
        if cp is not None:
            o, actx = cp.forward(li, qkv, plan)
        else:
            o, actx = attn_ops.forward(qkv, Hq, Hkv, hd, plan, need_grad=save)
        x2, T_o = layer["o"].forward(o, use_lora, residual=x)
        h2, rstd2 = ew.rmsnorm_fwd(x2, layer["ln2"], cfg.rms_norm_eps)
        if need_out or not hasattr(layer["mlp"], "recompute"):
            x3, mctx = layer["mlp"].forward(h2, x2, use_lora, save)
        else:
            x3, mctx = None, layer["mlp"].recompute(h2, x2, use_lora)
        if not save:
            return x3, None
        sv.x, sv.rstd1, sv.h1, sv.T_qkv, sv.attn_ctx, sv.o, sv.T_o = x, rstd1, h1, T_qkv, actx, o, T_o
        sv.x2, sv.rstd2, sv.mlp = x2, rstd2, mctx
        return x3, sv

    def forward(self, tokens: torch.Tensor, pos: torch.Tensor, gid: torch.Tensor, pid: torch.Tensor, S: int,
                use_lora: bool = True, save: bool = True, cp=None, x_in: torch.Tensor | None = None,
                recompute: str = "none") -> tuple[torch.Tensor, list[LayerSaved], dict]:
        """tokens int64 [M], pos/gid/pid int32 [M]; returns final-normed hidden [M,d] and saved state.

        With ``cp`` (a :class:`parallel.cp.ContextParallel`) ``tokens`` / ``pos`` hold this rank's shard of
        every packed row while ``gid`` / ``pid`` stay full-length; attention exchanges K/V with the peers.
        ``recompute``: "none" keeps every activation, "mlp" drops the feed-forward intermediates, "full" keeps only
        the layer inputs; :meth:`backward` rebuilds what is missing layer by layer.
        """
        cfg = self.cfg
        if recompute not in RECOMPUTE_MODES:
            raise ValueError(f"recompute must be one of {RECOMPUTE_MODES}")
        if recompute != "none" and cp is not None:
            raise ValueError("activation recompute is not combined with context parallelism (the K/V exchange of a "
                             "layer would have to run a second time on every rank)")
        x = ew.gather_rows(self.embed, tokens) if x_in is None else x_in     # x_in: activations from the previous stage
        plan = cp.make_plan(gid, pid) if cp is not None else attn_ops.make_plan(gid, pid, S, self.attn_impl)
        saved: list[LayerSaved] = []
        for li in range(len(self.layers)):
            if save and recompute == "full":
                x3, _ = self._layer_forward(li, x, pos, plan, use_lora, False, cp)
                saved.append(LayerSaved(recompute="full", x=x))
            else:
                x3, sv = self._layer_forward(li, x, pos, plan, use_lora, save, cp)
                if save:
                    if recompute == "mlp":
                        sv.recompute, sv.mlp = "mlp", None
                    saved.append(sv)
            x = x3
        final = {"cp": cp, "plan": plan, "use_lora": use_lora}
        if not self.is_last:
            return x, saved, final                                             # raw residual stream for the next stage
        hidden, rstd_f = ew.rmsnorm_fwd(x, self.final_norm, cfg.rms_norm_eps)
        final.update(x_last=x, rstd_f=rstd_f)
        return hidden, saved, final

    # -- backward ---------------------------------------------------------------------------
    def backward(self, dhidden: torch.Tensor, saved: list[LayerSaved], final: dict, pos: torch.Tensor
                 ) -> torch.Tensor | None:
        """Accumulate LoRA gradients given dLoss/dhidden [M,d] (bf16); returns the gradient w.r.t. the stage input
        (None on the first stage: the embedding is frozen)."""
        cfg = self.cfg
        Hq, Hkv, hd = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        dx = ew.rmsnorm_bwd(dhidden, final["x_last"], self.final_norm, final["rstd_f"]) if self.is_last else dhidden
        for li in range(len(self.layers) - 1, -1, -1):
            layer, sv = self.layers[li], saved[li]
            if sv.recompute == "full":       # rebuild this layer's activations from its input
                _, sv = self._layer_forward(li, sv.x, pos, final["plan"], final["use_lora"], True, None, need_out=False)
            elif sv.recompute == "mlp":      # rebuild the feed-forward intermediates from x2
                h2, _ = ew.rmsnorm_fwd(sv.x2, layer["ln2"], cfg.rms_norm_eps, want_rstd=False)
                mlp = layer["mlp"]
                sv.mlp = (mlp.recompute(h2, sv.x2, final["use_lora"]) if hasattr(mlp, "recompute")
                          else mlp.forward(h2, sv.x2, final["use_lora"], True)[1])
            # MLP
            dh2 = layer["mlp"].backward(dx, sv.mlp)
            dx2 = ew.rmsnorm_bwd(dh2, sv.x2, layer["ln2"], sv.rstd2, dres=dx)
            del dh2
            # attention
            do = layer["o"].backward(dx2, sv.o, sv.T_o)
            dqkv = final["cp"].backward(do, sv.attn_ctx) if final.get("cp") is not None else attn_ops.backward(do, sv.attn_ctx)
            del do
            ew.rope_(dqkv, pos, 0, Hq + Hkv, hd, cfg.rope_theta, inverse=True, **ew.rope_args(cfg, dqkv.device))
            if cfg.qk_norm:
                pre = torch.empty_like(dqkv)
                pre[:, : (Hq + Hkv) * hd] = sv.qk_pre
                ew.headnorm_bwd_(dqkv, pre, layer["q_norm"], sv.qk_rstd[0], 0, Hq, hd)
                ew.headnorm_bwd_(dqkv, pre, layer["k_norm"], sv.qk_rstd[1], Hq * hd, Hkv, hd)
                del pre
            need_dx = li > 0 or not self.is_first  # the embedding is frozen: layer 0 needs no input gradient
            dh1 = layer["qkv"].backward(dqkv, sv.h1, sv.T_qkv, need_dx=need_dx)
            del dqkv
            if need_dx:
                dx = ew.rmsnorm_bwd(dh1, sv.x, layer["ln1"], sv.rstd1, dres=dx2)
            saved[li] = None  # release this layer's activations
        return dx if not self.is_first else None
