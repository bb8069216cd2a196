"""Plain-PyTorch decoder + GRPO loss: the numerical oracle and the library baseline.

Everything here is ordinary differentiable PyTorch (matmul, softmax, autograd), runs on
CPU in fp32 for the oracle tests and on GPU in bf16 as the "library ops" baseline that
the sm_100a kernels are measured against.  Semantics restate the reference trainer:

* attention mask ``k <= q and (group[q] == group[k] or parent[q] == group[k])``
  (reference ``src/art/local/train.py:177-215``);
* selected-token log-prob from hidden states and the LM head (``train.py:245-281``);
* clipped-ratio GRPO loss with optional k3 KL term (``train.py:112-151``).

RoPE uses the packed ``input_pos`` (the position each token had when it was sampled)
unless ``compat_row_positions`` is set, in which case the index within the packed row is
used as the reference does.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from .config import ModelConfig
from .weights import LoraConfig, lora_key


def tree_attention_mask(group_ids: torch.Tensor, parent_ids: torch.Tensor) -> torch.Tensor:
    """[B,S] ids -> bool [B,S,S], True where query q may attend key k."""
    S = group_ids.shape[-1]
    causal = torch.ones(S, S, dtype=torch.bool, device=group_ids.device).tril()
    same = group_ids.unsqueeze(2) == group_ids.unsqueeze(1)
    parent = parent_ids.unsqueeze(2) == group_ids.unsqueeze(1)
    return causal & (same | parent)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


def rope_cos_sin(positions: torch.Tensor, head_dim: int, theta: float, cfg: ModelConfig | None = None
                 ) -> tuple[torch.Tensor, torch.Tensor]:
    """cos / sin [..., hd/2] of the rotary embedding; with ``cfg`` carrying a ``rope_scaling`` the frequencies and the
    attention scale come from ``cfg.rope_inv_freq()``."""
    if cfg is not None and cfg.rope_scaling is not None:
        inv_l, att = cfg.rope_inv_freq()
        inv = torch.tensor(inv_l, dtype=torch.float32, device=positions.device)
        ang = positions.float().unsqueeze(-1) * inv
        return ang.cos() * att, ang.sin() * att
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=positions.device, dtype=torch.float32) / head_dim))
    ang = positions.float().unsqueeze(-1) * inv  # [..., hd/2]
    return ang.cos(), ang.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [B,S,H,hd]; rotate-half convention (HF Qwen2/Llama)."""
    hd = x.shape[-1]
    x1, x2 = x[..., : hd // 2].float(), x[..., hd // 2:].float()
    c, s = cos.unsqueeze(-2), sin.unsqueeze(-2)
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


class ReferenceModel:
    """Functional decoder over a dict of HF-named base weights and PEFT-named LoRA params."""

    def __init__(self, cfg: ModelConfig, base: dict[str, torch.Tensor], lora: dict[str, torch.Tensor] | None = None,
                 lora_cfg: LoraConfig | None = None):
        self.cfg = cfg
        self.base = base
        self.lora = lora or {}
        self.lora_cfg = lora_cfg or LoraConfig()

    # -- building blocks ------------------------------------------------------------------
    def linear(self, x: torch.Tensor, layer: int, module: str, use_lora: bool = True) -> torch.Tensor:
        p = f"model.layers.{layer}.{module}"
        y = F.linear(x, self.base[p + ".weight"], self.base.get(p + ".bias"))
        ka = lora_key(layer, module, "A")
        if use_lora and ka in self.lora:
            a = self.lora[ka].to(x.dtype)
            b = self.lora[lora_key(layer, module, "B")].to(x.dtype)
            y = y + self.lora_cfg.scale * F.linear(F.linear(x, a), b)
        return y

    def attention(self, x, layer, cos, sin, mask, use_lora):
        cfg = self.cfg
        B, S, _ = x.shape
        q = self.linear(x, layer, "self_attn.q_proj", use_lora).view(B, S, cfg.num_heads, cfg.head_dim)
        k = self.linear(x, layer, "self_attn.k_proj", use_lora).view(B, S, cfg.num_kv_heads, cfg.head_dim)
        v = self.linear(x, layer, "self_attn.v_proj", use_lora).view(B, S, cfg.num_kv_heads, cfg.head_dim)
        if cfg.qk_norm:
            p = f"model.layers.{layer}.self_attn."
            q = rms_norm(q, self.base[p + "q_norm.weight"], cfg.rms_norm_eps)
            k = rms_norm(k, self.base[p + "k_norm.weight"], cfg.rms_norm_eps)
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        rep = cfg.num_heads // cfg.num_kv_heads
        q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
        k = k.repeat_interleave(rep, dim=1)
        v = v.repeat_interleave(rep, dim=1)
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=mask.unsqueeze(1))
        o = o.transpose(1, 2).reshape(B, S, cfg.q_size)
        return self.linear(o, layer, "self_attn.o_proj", use_lora)

    def mlp(self, x, layer, use_lora):
        cfg = self.cfg
        if not cfg.is_moe:
            g = self.linear(x, layer, "mlp.gate_proj", use_lora)
            u = self.linear(x, layer, "mlp.up_proj", use_lora)
            return self.linear(F.silu(g) * u, layer, "mlp.down_proj", use_lora)
        B, S, d = x.shape
        flat = x.reshape(-1, d)
        logits = F.linear(flat, self.base[f"model.layers.{layer}.mlp.gate.weight"])
        probs = logits.float().softmax(-1)
        topw, topi = probs.topk(cfg.num_experts_per_tok, dim=-1)
        if cfg.norm_topk_prob:
            topw = topw / topw.sum(-1, keepdim=True)
        out = torch.zeros_like(flat)
        for e in range(cfg.num_experts):
            tok, slot = (topi == e).nonzero(as_tuple=True)
            if tok.numel() == 0:
                continue
            xe = flat[tok]
            g = self.linear(xe, layer, f"mlp.experts.{e}.gate_proj", use_lora)
            u = self.linear(xe, layer, f"mlp.experts.{e}.up_proj", use_lora)
            ye = self.linear(F.silu(g) * u, layer, f"mlp.experts.{e}.down_proj", use_lora)
            out.index_add_(0, tok, ye * topw[tok, slot].unsqueeze(-1).to(ye.dtype))
        return out.view(B, S, d)

    # -- forward --------------------------------------------------------------------------
    def hidden_states(self, tokens: torch.Tensor, group_ids: torch.Tensor, parent_ids: torch.Tensor,
                      input_pos: torch.Tensor | None = None, use_lora: bool = True) -> torch.Tensor:
        """tokens/ids [B,S] -> final-norm hidden states [B,S,d]."""
        cfg = self.cfg
        B, S = tokens.shape
        pos = input_pos if input_pos is not None else torch.arange(S, device=tokens.device).expand(B, S)
        cos, sin = rope_cos_sin(pos, cfg.head_dim, cfg.rope_theta, cfg)
        mask = tree_attention_mask(group_ids, parent_ids)
        x = F.embedding(tokens, self.base["model.embed_tokens.weight"])
        for i in range(cfg.num_layers):
            p = f"model.layers.{i}."
            h = rms_norm(x, self.base[p + "input_layernorm.weight"], cfg.rms_norm_eps)
            x = x + self.attention(h, i, cos, sin, mask, use_lora)
            h = rms_norm(x, self.base[p + "post_attention_layernorm.weight"], cfg.rms_norm_eps)
            x = x + self.mlp(h, i, use_lora)
        return rms_norm(x, self.base["model.norm.weight"], cfg.rms_norm_eps)

    def logprobs(self, hidden: torch.Tensor, next_tokens: torch.Tensor, chunk: int = 1024) -> torch.Tensor:
        """Selected-token log-softmax without materialising [B,S,V] at once (fp32 softmax)."""
        w = self.base["lm_head.weight"]
        B, S, _ = hidden.shape
        outs = []
        for s in range(0, S, chunk):
            logits = F.linear(hidden[:, s:s + chunk], w).float()
            sel = logits.gather(-1, next_tokens[:, s:s + chunk].unsqueeze(-1)).squeeze(-1)
            outs.append(sel - torch.logsumexp(logits, dim=-1))
        return torch.cat(outs, dim=1)


def shift_left(t: torch.Tensor, pad) -> torch.Tensor:
    return F.pad(t[:, 1:], (0, 1), value=pad)


def grpo_loss(new_logprobs: torch.Tensor, packed: dict[str, torch.Tensor], epsilon: float = 0.2,
              epsilon_high: float | None = None, beta: float = 0.0,
              ref_logprobs: torch.Tensor | None = None) -> tuple[torch.Tensor, dict[str, torch.Tensor]]:
    """Clipped-ratio policy loss (+ beta * k3 KL), averaged over assistant tokens."""
    if epsilon_high is None:
        epsilon_high = epsilon
    old = shift_left(packed["logprobs"], 0.0)
    adv = shift_left(packed["advantages"], 0.0)
    mask = shift_left(packed["assistant_mask"], False).to(new_logprobs.dtype)
    wts = shift_left(packed["weights"], 0.0)
    old = torch.where(torch.isnan(old), new_logprobs.detach(), old)
    ratio = torch.exp(new_logprobs - old)
    pg = -torch.min(ratio * adv, torch.clip(ratio, 1 - epsilon, 1 + epsilon_high) * adv)
    if ref_logprobs is not None:
        diff = ref_logprobs - new_logprobs
        kl = torch.exp(diff) - diff - 1.0
    else:
        kl = torch.zeros_like(pg)
    denom = mask.sum() + 1e-6
    policy_loss = (pg * wts * mask).sum() / denom
    kl_mean = (kl * wts * mask).sum() / denom
    return policy_loss + beta * kl_mean, {"policy_loss": policy_loss.detach(), "kl_div": kl_mean.detach()}


def reference_train_step(model: ReferenceModel, packed: dict[str, torch.Tensor], optimizer: torch.optim.Optimizer,
                         lr: float, beta: float = 0.0, epsilon: float = 0.2, epsilon_high: float | None = None,
                         max_grad_norm: float = 0.1, compat_row_positions: bool = False) -> dict[str, float]:
    """One optimizer step over all rows in ``packed`` (rows are summed into one gradient)."""
    for g in optimizer.param_groups:
        g["lr"] = lr
    pos = None if compat_row_positions else packed["input_pos"]
    hidden = model.hidden_states(packed["tokens"], packed["group_ids"], packed["parent_ids"], pos)
    nxt = shift_left(packed["tokens"], 0)
    new_lp = model.logprobs(hidden, nxt)
    ref_lp = None
    if beta > 0:
        with torch.no_grad():
            ref_h = model.hidden_states(packed["tokens"], packed["group_ids"], packed["parent_ids"], pos, use_lora=False)
            ref_lp = model.logprobs(ref_h, nxt)
    loss, metrics = grpo_loss(new_lp, packed, epsilon, epsilon_high, beta, ref_lp)
    optimizer.zero_grad(set_to_none=True)
    loss.backward()
    params = [p for g in optimizer.param_groups for p in g["params"]]
    gnorm = torch.nn.utils.clip_grad_norm_(params, max_grad_norm)
    optimizer.step()
    out = {"loss": float(loss), "grad_norm": float(gnorm), "policy_loss": float(metrics["policy_loss"]), "learning_rate": lr}
    if beta > 0:
        out["kl_div"] = float(metrics["kl_div"])
    return out
