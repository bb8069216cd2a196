"""Tensor-parallel dense decoder (Megatron layout with token-sharded activations) on the fused
all-gather->GEMM / GEMM->reduce-scatter kernels.

Rank ``p`` of ``P`` holds the q/k/v heads ``[p*H/P, (p+1)*H/P)``, the matching columns of ``o_proj``,
and a 1/P slice of the feed-forward width.  The residual stream, both RMSNorms, the LM head and the
loss work on the rank's contiguous ``M/P`` token segment; only attention and the MLP activation
see all ``M`` tokens (for the local heads / columns).  Per layer and direction there are exactly two
all-gather->GEMM and two GEMM->reduce-scatter launches and no other collective:

    forward   qkv = AG->GEMM(h1)      x2 = GEMM->RS(attn) + x       gate|up = AG->GEMM(h2)      x3 = GEMM->RS(act) + x2
    backward  d act = AG->GEMM(dx3)   d h2 = GEMM->RS(d gate|up)    d attn = AG->GEMM(dx2)      d h1 = GEMM->RS(d qkv)

LoRA: a column-parallel linear keeps ``A`` whole (its low-rank activations ``T = X A^T`` are
computed on the token shard and gathered together with ``X``) and the local rows of ``B``; a
row-parallel linear keeps the local columns of ``A`` and ``B`` whole, and its partial ``T_p B^T`` is
summed by the reduce-scatter.  Every rank stores the full fp32 LoRA masters; each computes the
gradient of the slices it owns and a partial gradient of the replicated factors, and one SUM
all-reduce of the flat gradient buffer over the tensor-parallel group completes both.

The reference has no tensor parallelism of its own (``src/art/dev/engine.py:27`` forwards
``tensor_parallel_size`` to the inference library); this is the trainer side of the "TP2 x DP4" layout.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..ops import attention as attn_ops
from ..ops import elementwise as ew
from ..ops.gemm import gemm_tn
from .config import ModelConfig
from .native import LORA_KPAD, LoraFlat, lora_wgrad
from .weights import LoraConfig, lora_key


@dataclass
class _TPMember:
    rows: torch.Tensor        # rows of this module inside the LOCAL fused weight
    slot: int
    a_view: torch.Tensor      # full fp32 masters / gradients
    b_view: torch.Tensor
    ga_view: torch.Tensor
    gb_view: torch.Tensor
    own: torch.Tensor         # column-parallel: rows of B owned by this rank; row-parallel: columns of A


class _TPLinear:
    def __init__(self, members: list[_TPMember], r: int, scale: float):
        self.members, self.r, self.scale = members, r, scale
        self.active = len(members) > 0
        self.kpad = LORA_KPAD

    def zero_grad(self):
        if self.active:
            self.dA_acc.zero_()
            self.dB_acc.zero_()


class ColumnParallelLinear(_TPLinear):
    """``Y[:, local cols] = gather(X) W_p^T``; weight ``[N_p, K]`` (local output rows)."""

    def __init__(self, tp, weight, bias, members, r, scale):
        super().__init__(members, r, scale)
        self.tp = tp
        self.W = weight.contiguous()
        self.WT = weight.t().contiguous()        # [K, N_p]
        self.bias = bias.float().contiguous() if bias is not None else None
        N, K = self.W.shape
        dev, bf = self.W.device, torch.bfloat16
        if self.active:
            self.A_cat = torch.zeros(self.kpad, K, dtype=bf, device=dev)
            self.B_cat = torch.zeros(N, self.kpad, dtype=bf, device=dev)
            self.A_catT = torch.zeros(K, self.kpad, dtype=bf, device=dev)
            self.B_catT = torch.zeros(self.kpad, N, dtype=bf, device=dev)
            self.dA_acc = torch.zeros(K, self.kpad, dtype=torch.float32, device=dev)
            self.dB_acc = torch.zeros(N, self.kpad, dtype=torch.float32, device=dev)

    def refresh(self):
        if not self.active:
            return
        r = self.r
        for m in self.members:
            c0 = m.slot * r
            self.A_cat[c0:c0 + r] = m.a_view
            self.B_cat[m.rows, c0:c0 + r] = (m.b_view[m.own] * self.scale).to(torch.bfloat16)
        self.A_catT.copy_(self.A_cat.t())
        self.B_catT.copy_(self.B_cat.t())

    def export_grads(self):
        if not self.active:
            return
        r = self.r
        for m in self.members:
            c0 = m.slot * r
            m.ga_view.copy_(self.dA_acc[:, c0:c0 + r].t())          # partial: summed over the group
            m.gb_view.zero_()
            m.gb_view[m.own] = self.dB_acc[m.rows, c0:c0 + r] * self.scale

    def forward(self, h_shard, use_lora=True, swiglu_out=None, save=True):
        """``h_shard`` may already BE the view returned by ``tp.ag_input(K)`` (the producer wrote into it)."""
        tp = self.tp
        K = self.W.shape[1]
        dst = tp.ag_input(K)
        if h_shard.data_ptr() != dst.data_ptr():
            dst.copy_(h_shard)
        lora = self.active and use_lora
        if lora:
            gemm_tn(h_shard, self.A_cat, out=tp.ag_t_input())
        y, x_full, t_full = tp.ag_gemm(K, self.W, b2=self.B_cat if lora else None, swiglu_out=swiglu_out, bias=self.bias)
        if not save:
            return y, None
        return y, (x_full.clone(), t_full.clone() if lora else None)

    def backward(self, dy, saved, need_dx=True, dres_shard=None):
        x_full, t_full = saved
        if self.active and t_full is not None:
            dT = gemm_tn(dy, self.B_catT)
            lora_wgrad(self.dA_acc, x_full, dT)
            lora_wgrad(self.dB_acc, dy, t_full)
            if need_dx:
                return self.tp.gemm_rs(dy, self.WT, a2=dT, b2=self.A_catT, residual=dres_shard)
            return None
        return self.tp.gemm_rs(dy, self.WT, residual=dres_shard) if need_dx else None


class RowParallelLinear(_TPLinear):
    """``Y_shard = reduce_scatter(X_p W_p^T)``; weight ``[N, K_p]`` (local input columns)."""

    def __init__(self, tp, weight, members, r, scale):
        super().__init__(members, r, scale)
        self.tp = tp
        self.W = weight.contiguous()
        self.WT = weight.t().contiguous()        # [K_p, N]
        N, K = self.W.shape
        dev, bf = self.W.device, torch.bfloat16
        if self.active:
            self.A_cat = torch.zeros(self.kpad, K, dtype=bf, device=dev)
            self.B_cat = torch.zeros(N, self.kpad, dtype=bf, device=dev)
            self.A_catT = torch.zeros(K, self.kpad, dtype=bf, device=dev)
            self.B_catT = torch.zeros(self.kpad, N, dtype=bf, device=dev)
            self.dA_acc = torch.zeros(K, self.kpad, dtype=torch.float32, device=dev)
            self.dB_acc = torch.zeros(N, self.kpad, dtype=torch.float32, device=dev)

    def refresh(self):
        if not self.active:
            return
        r = self.r
        for m in self.members:
            c0 = m.slot * r
            self.A_cat[c0:c0 + r] = m.a_view[:, m.own]
            self.B_cat[m.rows, c0:c0 + r] = (m.b_view * self.scale).to(torch.bfloat16)
        self.A_catT.copy_(self.A_cat.t())
        self.B_catT.copy_(self.B_cat.t())

    def export_grads(self):
        if not self.active:
            return
        r = self.r
        for m in self.members:
            c0 = m.slot * r
            m.ga_view.zero_()
            m.ga_view[:, m.own] = self.dA_acc[:, c0:c0 + r].t()
            m.gb_view.copy_(self.dB_acc[m.rows, c0:c0 + r] * self.scale)   # partial: summed over the group

    def forward(self, x_p, residual_shard, use_lora=True, save=True):
        if self.active and use_lora:
            T = gemm_tn(x_p, self.A_cat)
            y = self.tp.gemm_rs(x_p, self.W, a2=T, b2=self.B_cat, residual=residual_shard)
            return y, (T if save else None)
        return self.tp.gemm_rs(x_p, self.W, residual=residual_shard), None

    def backward(self, dy_shard, x_p, T, swiglu_gu=None):
        """``swiglu_gu``: this linear's input was ``silu(gate) * up``; return d(gate|up) instead of d(input).
        ``dy_shard`` may already be the view returned by ``tp.ag_input(N)``."""
        tp = self.tp
        N = self.W.shape[0]
        dst = tp.ag_input(N)
        if dy_shard.data_ptr() != dst.data_ptr():
            dst.copy_(dy_shard)
        lora = self.active and T is not None
        if lora:
            gemm_tn(dy_shard, self.B_catT, out=tp.ag_t_input())
        dx_p, dy_full, dT_full = tp.ag_gemm(N, self.WT, b2=self.A_catT if lora else None, swiglu_bwd_gu=swiglu_gu)
        if lora:
            lora_wgrad(self.dA_acc, x_p, dT_full)
            lora_wgrad(self.dB_acc, dy_full, T)
        return dx_p


@dataclass
class TPLayerSaved:
    x: torch.Tensor = None
    rstd1: torch.Tensor = None
    qkv_in: tuple = None
    attn_ctx: object = None
    o: torch.Tensor = None
    T_o: torch.Tensor = None
    x2: torch.Tensor = None
    rstd2: torch.Tensor = None
    gu_in: tuple = None
    gu: torch.Tensor = None
    hact: torch.Tensor = None
    T_d: torch.Tensor = None
    qk_pre: torch.Tensor = None
    qk_rstd: tuple = None


class TPDecoder:
    """Dense decoder sharded over a tensor-parallel group; same forward/backward contract as ``NativeDecoder`` except
    that ``tokens`` is this rank's contiguous token segment and ``pos`` / ``gid`` / ``pid`` cover all ``M`` tokens."""

    def __init__(self, cfg: ModelConfig, base: dict[str, torch.Tensor], lora_cfg: LoraConfig,
                 lora_init: dict[str, torch.Tensor], tp, device="cuda"):
        if cfg.is_moe:
            raise ValueError("tensor parallelism covers the dense model family; use expert parallelism for MoE")
        P, p = tp.world, tp.rank
        if cfg.num_heads % P or cfg.num_kv_heads % P or cfg.intermediate_size % (16 * P):
            raise ValueError("heads and feed-forward width must divide over the tensor-parallel group")
        self.cfg, self.lora_cfg, self.tp = cfg, lora_cfg, tp
        self.device = dev = torch.device(device)
        ew.rope_args(cfg, dev)               # frequency table of a scaled rotary embedding, built outside the step
        bf = torch.bfloat16
        self.embed = base["model.embed_tokens.weight"].to(dev, bf).contiguous()
        self.lm_head = base["lm_head.weight"].to(dev, bf).contiguous()
        V, d = self.lm_head.shape
        self.lm_head_t = torch.zeros(d, (V + 7) // 8 * 8, dtype=bf, device=dev)
        self.lm_head_t[:, :V] = self.lm_head.t()
        self.final_norm = base["model.norm.weight"].to(dev, bf).contiguous()
        self.flat = LoraFlat(cfg, lora_cfg, lora_init, dev)
        r, s, hd = lora_cfg.r, lora_cfg.scale, cfg.head_dim
        self.Hq, self.Hkv = cfg.num_heads // P, cfg.num_kv_heads // P
        ql, kvl, Fl = self.Hq * hd, self.Hkv * hd, cfg.intermediate_size // P
        ar = lambda a, b: torch.arange(a, b, device=dev)   # noqa: E731
        q_own, kv_own, f_own = ar(p * ql, (p + 1) * ql), ar(p * kvl, (p + 1) * kvl), ar(p * Fl, (p + 1) * Fl)
        fidx = torch.arange(Fl, device=dev)
        gate_rows = (fidx // 16) * 32 + fidx % 16
        self.layers = []
        for i in range(cfg.num_layers):
            pre = f"model.layers.{i}."

            def W(name):
                return base[pre + name + ".weight"].to(dev, bf)

            def members(specs):
                out = []
                for slot, (module, rows, own) in enumerate(specs):
                    ka = lora_key(i, module, "A")
                    if ka in self.flat.views:
                        kb = lora_key(i, module, "B")
                        out.append(_TPMember(rows, slot, self.flat.views[ka], self.flat.views[kb],
                                             self.flat.grad_views[ka], self.flat.grad_views[kb], own))
                return out

            wqkv = torch.cat([W("self_attn.q_proj")[q_own], W("self_attn.k_proj")[kv_own], W("self_attn.v_proj")[kv_own]], 0)
            bqkv = None
            if cfg.qkv_bias:
                bqkv = torch.cat([base[pre + "self_attn.q_proj.bias"].to(dev)[q_own],
                                  base[pre + "self_attn.k_proj.bias"].to(dev)[kv_own],
                                  base[pre + "self_attn.v_proj.bias"].to(dev)[kv_own]])
            qkv = ColumnParallelLinear(tp, wqkv, bqkv, members([
                ("self_attn.q_proj", ar(0, ql), q_own), ("self_attn.k_proj", ar(ql, ql + kvl), kv_own),
                ("self_attn.v_proj", ar(ql + kvl, ql + 2 * kvl), kv_own)]), r, s)
            o = RowParallelLinear(tp, W("self_attn.o_proj")[:, q_own], members([("self_attn.o_proj", ar(0, d), q_own)]), r, s)
            wgu = ew.interleave_gate_up(W("mlp.gate_proj")[f_own], W("mlp.up_proj")[f_own])
            gu = ColumnParallelLinear(tp, wgu, None, members([("mlp.gate_proj", gate_rows, f_own),
                                                               ("mlp.up_proj", gate_rows + 16, f_own)]), r, s)
            down = RowParallelLinear(tp, W("mlp.down_proj")[:, f_own], members([("mlp.down_proj", ar(0, d), f_own)]), r, s)
            layer = {"qkv": qkv, "o": o, "gu": gu, "down": down,
                     "ln1": base[pre + "input_layernorm.weight"].to(dev, bf).contiguous(),
                     "ln2": base[pre + "post_attention_layernorm.weight"].to(dev, bf).contiguous()}
            if cfg.qk_norm:
                layer["q_norm"] = base[pre + "self_attn.q_norm.weight"].to(dev, bf).contiguous()
                layer["k_norm"] = base[pre + "self_attn.k_norm.weight"].to(dev, bf).contiguous()
            self.layers.append(layer)
        self.Fl = Fl
        self.refresh_lora()

    def linears(self):
        for layer in self.layers:
            for k in ("qkv", "o", "gu", "down"):
                yield layer[k]

    def refresh_lora(self):
        for lin in self.linears():
            lin.refresh()

    def zero_grad(self):
        for lin in self.linears():
            lin.zero_grad()

    def export_grads(self):
        for lin in self.linears():
            lin.export_grads()

    def forward(self, tokens, pos, gid, pid, S, use_lora=True, save=True, cp=None):
        cfg, Hq, Hkv, hd = self.cfg, self.Hq, self.Hkv, self.cfg.head_dim
        x = ew.gather_rows(self.embed, tokens)                     # [m_seg, d]
        plan = attn_ops.make_plan(gid, pid, S, "native")
        saved = []
        for layer in self.layers:
            sv = TPLayerSaved()
            # the norm writes its output straight into this rank's rows of the gathered operand
            h1, rstd1 = ew.rmsnorm_fwd(x, layer["ln1"], cfg.rms_norm_eps, out=self.tp.ag_input(cfg.hidden_size))
            qkv, qkv_in = layer["qkv"].forward(h1, use_lora, save=save)
            if cfg.qk_norm:
                if save:
                    sv.qk_pre = qkv[:, : (Hq + Hkv) * hd].clone()
                rq = ew.headnorm_fwd_(qkv, layer["q_norm"], 0, Hq, hd, cfg.rms_norm_eps)
                rk = ew.headnorm_fwd_(qkv, layer["k_norm"], Hq * hd, Hkv, hd, cfg.rms_norm_eps)
                sv.qk_rstd = (rq, rk)
            ew.rope_(qkv, pos, 0, Hq + Hkv, hd, cfg.rope_theta, **ew.rope_args(cfg, qkv.device))
            o, actx = attn_ops.forward(qkv, Hq, Hkv, hd, plan, need_grad=save)
            x2, T_o = layer["o"].forward(o, x, use_lora, save=save)
            h2, rstd2 = ew.rmsnorm_fwd(x2, layer["ln2"], cfg.rms_norm_eps, out=self.tp.ag_input(cfg.hidden_size))
            hact = torch.empty((qkv.shape[0], self.Fl), dtype=x.dtype, device=x.device)
            gu, gu_in = layer["gu"].forward(h2, use_lora, swiglu_out=hact, save=save)
            x3, T_d = layer["down"].forward(hact, x2, use_lora, save=save)
            if save:
                sv.x, sv.rstd1, sv.qkv_in, sv.attn_ctx, sv.o, sv.T_o = x, rstd1, qkv_in, actx, o, T_o
                sv.x2, sv.rstd2, sv.gu_in, sv.gu, sv.hact, sv.T_d = x2, rstd2, gu_in, gu, hact, T_d
                saved.append(sv)
            x = x3
        hidden, rstd_f = ew.rmsnorm_fwd(x, self.final_norm, cfg.rms_norm_eps)
        return hidden, saved, {"x_last": x, "rstd_f": rstd_f}

    def backward(self, dhidden, saved, final, pos):
        cfg, Hq, Hkv, hd = self.cfg, self.Hq, self.Hkv, self.cfg.head_dim
        # every residual-stream gradient is the input of the next all-gather->GEMM: the norm backward writes it straight
        # into this rank's rows of the gathered operand (the buffers alternate per call, so the previous one, still
        # needed as the residual term of the following norm backward, stays intact)
        d = cfg.hidden_size
        dx = ew.rmsnorm_bwd(dhidden, final["x_last"], self.final_norm, final["rstd_f"], out=self.tp.ag_input(d))
        for li in range(cfg.num_layers - 1, -1, -1):
            layer, sv = self.layers[li], saved[li]
            # d(gate|up) [M, 2F/P]: the SwiGLU backward sits in the epilogue of the down projection's data-gradient GEMM
            dgu = layer["down"].backward(dx, sv.hact, sv.T_d, swiglu_gu=sv.gu)
            dh2 = layer["gu"].backward(dgu, sv.gu_in)                          # [m_seg, d]
            del dgu
            dx2 = ew.rmsnorm_bwd(dh2, sv.x2, layer["ln2"], sv.rstd2, dres=dx, out=self.tp.ag_input(d))
            del dh2
            do = layer["o"].backward(dx2, sv.o, sv.T_o)                        # [M, q/P]
            dqkv = attn_ops.backward(do, sv.attn_ctx)
            del do
            ew.rope_(dqkv, pos, 0, Hq + Hkv, hd, cfg.rope_theta, inverse=True, **ew.rope_args(cfg, dqkv.device))
            if cfg.qk_norm:
                pre = torch.empty_like(dqkv)
                pre[:, : (Hq + Hkv) * hd] = sv.qk_pre
                ew.headnorm_bwd_(dqkv, pre, layer["q_norm"], sv.qk_rstd[0], 0, Hq, hd)
                ew.headnorm_bwd_(dqkv, pre, layer["k_norm"], sv.qk_rstd[1], Hq * hd, Hkv, hd)
                del pre
            need_dx = li > 0
            dh1 = layer["qkv"].backward(dqkv, sv.qkv_in, need_dx=need_dx)
            del dqkv
            if need_dx:
                dx = ew.rmsnorm_bwd(dh1, sv.x, layer["ln1"], sv.rstd1, dres=dx2, out=self.tp.ag_input(d))
            saved[li] = None
