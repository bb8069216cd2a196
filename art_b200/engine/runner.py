"""Model execution for the rollout engine.

``NativeRunner``    sm_100a path.  Shares the frozen base weights with the trainer's
                    :class:`models.native.NativeDecoder` when both live in one process, holds
                    ``max_loras`` resident adapters side by side in the extra-K operands of
                    every projection (adapter ``a`` owns a column range of ``T = X A_all^T``; a
                    per-row mask keeps only the requesting adapter's columns, so one GEMM serves
                    a batch that mixes adapters and the base model), writes K/V into the paged
                    cache, and samples with the fused LM-head sampler.  Decode runs several steps
                    back to back on the device before the host looks at the tokens.
``ReferenceRunner`` plain PyTorch, no KV cache (recomputes the prefix); used for CPU tests of
                    the scheduler / server / backend and as a numerical oracle.

Both return ``(token_ids, logprobs)`` as Python lists so the scheduler is device-agnostic.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass

import torch

from ..models.config import ModelConfig
from ..models.weights import LoraConfig, lora_key


@dataclass
class LogitProc:
    """Per-request logit processing that needs the materialised logits of a step (not the fused sampler)."""
    n_prompt: int
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    logit_bias: dict | None = None
    top_logprobs: int = 0
    grammar: object | None = None       # grammar.GrammarState / AllowedSet: only tokens of its mask may be drawn
    min_tokens: int = 0                 # tokens of `end_ids` are excluded while the output is shorter than this
    end_ids: tuple = ()
    bad_words_ids: list | None = None   # token sequences whose last token is excluded once the others have been emitted

    @property
    def edits(self) -> bool:
        return (self.repetition_penalty != 1.0 or self.presence_penalty != 0.0 or self.frequency_penalty != 0.0
                or bool(self.logit_bias) or self.min_tokens > 0 or bool(self.bad_words_ids))


def apply_token_mask(logits: torch.Tensor, grammars: list) -> torch.Tensor:
    """Sets the logits of tokens outside each row's grammar mask to -1e30 (finite: the samplers scale logits by an
    inverse temperature that may be 0), in place.  ``logits`` [M, V] fp32; ``grammars[i]`` is None or a
    ``grammar.GrammarState``.  Ids past the tokenizer's vocabulary (padding rows of the embedding) are never allowed; a
    row whose mask is empty is left alone.  Plain PyTorch: the path is taken one decode step at a time and only by
    requests with structured outputs."""
    V = logits.shape[1]
    for i, g in enumerate(grammars):
        if g is None:
            continue
        m = torch.from_numpy(g.allowed())
        if not bool(m[:V].any()):
            continue
        allowed = torch.zeros(V, dtype=torch.bool)
        allowed[: min(V, m.numel())] = m[:V]
        logits[i].masked_fill_(~allowed.to(logits.device), -1e30)
    return logits


@dataclass(slots=True)
class SeqView:
    """What a runner needs to know about one scheduled sequence."""
    tokens: list[int]          # prompt + generated so far
    num_cached: int            # tokens whose KV is already in the cache (multiple of block_size)
    blocks: list[int]          # block table
    adapter: int               # adapter slot, -1 = base model
    temperature: float
    seed: int
    step: int                  # number of tokens generated so far (mixes into the sampling seed)
    top_p: float = 1.0         # nucleus mass (>= 1: off)
    top_k: int = -1            # keep the k most likely tokens (<= 0: off)
    min_p: float = 0.0         # keep tokens at least min_p times as likely as the most likely one (<= 0: off)
    proc: LogitProc | None = None   # penalties / logit_bias / top_logprobs: the step materialises fp32 logits
    upto: int | None = None    # chunked prefill: compute KV for tokens[num_cached:upto] only and sample nothing

    @property
    def partial(self) -> bool:
        return self.upto is not None and self.upto < len(self.tokens)

    @property
    def restricted(self) -> bool:
        return self.temperature > 0 and (self.top_p < 1.0 or self.top_k > 0 or self.min_p > 0)


def _mix_seed(seed: int, step: int) -> int:
    return (seed * 0x9E3779B1 + step * 0x85EBCA77 + 0x165667B1) & 0xFFFFFFFF


# ------------------------------------------------------------------------------- reference
class ReferenceRunner:
    def __init__(self, cfg: ModelConfig, base: dict[str, torch.Tensor], lora_cfg: LoraConfig, max_loras: int = 4,
                 device: str | torch.device = "cpu"):
        from ..models.reference import ReferenceModel

        self.cfg, self.lora_cfg, self.device = cfg, lora_cfg, torch.device(device)
        self.base = {k: v.to(self.device) for k, v in base.items()}
        self.adapters: list[dict[str, torch.Tensor] | None] = [None] * max_loras
        self._model = ReferenceModel(cfg, self.base, {}, lora_cfg)
        self._top = None
        self.last_top_logprobs: list | None = None      # [step][seq] -> None or [(token, logprob)] of the last call

    def set_adapter(self, slot: int, state: dict[str, torch.Tensor] | None) -> None:
        self.adapters[slot] = None if state is None else {k: v.detach().to(self.device).float() for k, v in state.items()}

    def _next(self, sv: SeqView) -> tuple[int, float]:
        m = self._model
        m.lora = self.adapters[sv.adapter] if sv.adapter >= 0 and self.adapters[sv.adapter] is not None else {}
        toks = torch.tensor([sv.tokens], device=self.device)
        z = torch.zeros_like(toks)
        with torch.no_grad():
            h = m.hidden_states(toks, z, z, None)[:, -1]
            logits = (h.float() @ self.base["lm_head.weight"].float().t())[0]
        self._top = None
        if sv.proc is not None:
            from ..ops.paged import build_logit_edits, logit_adjust_, top_logprobs

            if sv.proc.edits:
                logits = logit_adjust_(logits[None].clone(), build_logit_edits([(sv.proc, sv.tokens)]))[0]
            if sv.proc.grammar is not None:
                logits = apply_token_mask(logits[None].clone(), [sv.proc.grammar])[0]
            if sv.proc.top_logprobs > 0:
                it = torch.tensor([0.0 if sv.temperature <= 0 else 1.0 / sv.temperature])
                ti, tl = top_logprobs(logits[None].cpu(), it, sv.proc.top_logprobs)
                self._top = list(zip(ti[0].tolist(), tl[0].tolist()))
        if sv.temperature <= 0:
            lp = torch.log_softmax(logits, -1)
            t = int(lp.argmax())
            return t, float(lp[t])
        lp = torch.log_softmax(logits / sv.temperature, -1)
        probs = lp.exp()
        if sv.restricted:      # top-k, then top-p on the rest; the log-prob stays that of the full distribution
            from ..ops.paged import reference_restrict

            probs = probs * reference_restrict(logits / sv.temperature, sv.top_k, sv.top_p, sv.min_p)
        g = torch.Generator(device="cpu").manual_seed(_mix_seed(sv.seed, sv.step))
        t = int(torch.multinomial(probs.cpu(), 1, generator=g))
        return t, float(lp[t])

    def score(self, tokens: list[int], n_prompt: int, adapter: int) -> list[float]:
        m = self._model
        m.lora = self.adapters[adapter] if adapter >= 0 and self.adapters[adapter] is not None else {}
        toks = torch.tensor([tokens], device=self.device)
        z = torch.zeros_like(toks)
        with torch.no_grad():
            h = m.hidden_states(toks, z, z, None)[0, n_prompt - 1: len(tokens) - 1]
            lp = torch.log_softmax(h.float() @ self.base["lm_head.weight"].float().t(), -1)
        tgt = torch.tensor(tokens[n_prompt:], device=self.device)
        return lp.gather(-1, tgt.unsqueeze(-1)).squeeze(-1).tolist()

    def prefill(self, seqs: list[SeqView]) -> tuple[list[int], list[float]]:
        out, tops = [], []
        for s in seqs:
            if s.partial:                # no KV cache to fill here: the last chunk recomputes the whole prefix
                out.append((None, None))
                tops.append(None)
                continue
            out.append(self._next(s))
            tops.append(self._top)
        self.last_top_logprobs = [tops]
        return [o[0] for o in out], [o[1] for o in out]

    def decode(self, seqs: list[SeqView], n_steps: int) -> tuple[list[list[int]], list[list[float]]]:
        toks: list[list[int]] = []
        lps: list[list[float]] = []
        work = [SeqView(list(s.tokens), s.num_cached, s.blocks, s.adapter, s.temperature, s.seed, s.step, s.top_p, s.top_k,
                        s.min_p, s.proc) for s in seqs]
        self.last_top_logprobs = []
        for _ in range(n_steps):
            step_t, step_l, step_top = [], [], []
            for s in work:
                t, lp = self._next(s)
                s.tokens.append(t)
                s.step += 1
                step_t.append(t)
                step_l.append(lp)
                step_top.append(self._top)
            toks.append(step_t)
            lps.append(step_l)
            self.last_top_logprobs.append(step_top)
        return toks, lps


# ---------------------------------------------------------------------------------- native
# CTA-pair GEMMs at decode time: "1" = every projection, "wide" = only the unsplit (gate|up) ones, "0" = none
_TWO_CTA_MODE = os.environ.get("ARTB_DECODE_2CTA", "1")
TWO_CTA_DECODE = _TWO_CTA_MODE != "0"
# Decode-time form of the projections with a short reduction (q|k|v, o: K = hidden size):
#   "narrow"  one pass of 128 x 64 tiles (one wave of CTAs, each streaming its 64 weight rows over all of K), the
#             multi-LoRA update as extra K after a skinny shrink; no fp32 workspace, no finalize pass, no expand GEMM
#   "splitk"  split-K on CTA pairs into an fp32 workspace + finalize + LoRA expand GEMM
_DECODE_PLAN = os.environ.get("ARTB_DECODE_PLAN", "splitk")   # measured: 9.37 ms (splitk) vs 9.52 ms (narrow) per 256-sequence step at 7B
NARROW_MAX_K = 4096


class EngineLinear:
    """A frozen projection plus ``max_loras`` adapter slots.

    The weight is stored as ``W_ext = [W ; A_all]`` (the stacked shrink factors of all resident
    adapters are extra output rows), so at decode time one weight-streaming GEMM yields both the
    base product and ``T = X A_all^T``; after the per-row slot mask a small second GEMM adds
    ``T (sB_all)^T``.  Large-M (prefill) calls use the extra-K form instead.
    """

    def __init__(self, lin, member_rows: list[tuple], r: int, max_loras: int, ws_holder: dict):
        """``member_rows``: ``(module, rows)`` or ``(module, rows, out_slice, in_slice)``; the slices select this
        tensor-parallel rank's part of the adapter's ``B`` rows / ``A`` columns (None = all)."""
        W = lin.W
        N, K = W.shape
        self.N, self.K = N, K
        self.members = member_rows
        self.r = r
        self.cols = len(member_rows) * r
        self.kpad = max(64, (max_loras * self.cols + 63) // 64 * 64)
        self.W_ext = torch.zeros(N + self.kpad, K, dtype=torch.bfloat16, device=W.device)
        self.W_ext[:N] = W
        lin.W = self.W_ext[:N]                 # the trainer keeps using the same storage: no second copy of W
        self.W = self.W_ext[:N]
        self.A_all = self.W_ext[N:]
        self.B_all = torch.zeros(N, self.kpad, dtype=torch.bfloat16, device=W.device)
        self.B_T = torch.zeros(self.kpad, N, dtype=torch.bfloat16, device=W.device)    # same values, transposed (decode)
        self.bias_ext = None
        if lin.bias is not None:
            self.bias_ext = torch.zeros(N + self.kpad, dtype=torch.float32, device=W.device)
            self.bias_ext[:N] = lin.bias
        self.ws_holder = ws_holder

    def load_slot(self, slot: int, layer: int, state: dict[str, torch.Tensor] | None, scale: float) -> None:
        c0 = slot * self.cols
        self.A_all[c0:c0 + self.cols].zero_()
        self.B_all[:, c0:c0 + self.cols].zero_()
        self.B_T[c0:c0 + self.cols].zero_()
        if state is None:
            return
        for j, member in enumerate(self.members):
            module, rows = member[0], member[1]
            out_slice, in_slice = (member[2], member[3]) if len(member) > 2 else (None, None)
            ka = lora_key(layer, module, "A")
            if ka not in state:
                continue
            a, b = state[ka], state[lora_key(layer, module, "B")]
            if in_slice is not None:
                a = a[:, in_slice]
            if out_slice is not None:
                b = b[out_slice]
            c = c0 + j * self.r
            self.A_all[c:c + self.r] = a           # device-to-device copy straight from the trainer's master buffer
            self.B_all[rows, c:c + self.r] = (b * scale).to(torch.bfloat16)
            self.B_T[c:c + self.r, rows] = (b * scale).to(torch.bfloat16).t()

    def _ws(self, M: int, N: int, device) -> torch.Tensor:
        ws = self.ws_holder.get("ws")
        if ws is None or ws.shape[0] < M or ws.shape[1] < N:
            ws = torch.zeros((max(M, 512), max(N, 40960)), dtype=torch.float32, device=device)
            self.ws_holder["ws"] = ws
        return ws

    def partial_sums(self, x, any_lora: bool) -> torch.Tensor:
        """Decode-time product left as fp32 partial sums in the shared workspace: columns ``[0, N)`` hold ``X W^T`` and,
        with ``any_lora``, columns ``[N, N + kpad)`` the stacked shrink products ``X A_all^T``.  The fused consumers
        (``ops.paged.decode_finalize_norm`` / ``decode_finalize_qkv``) finish the projection and re-zero the columns."""
        from ..ops.gemm import gemm_splitk_, plan_small_m

        M, N = x.shape[0], self.N
        Next = N + self.kpad if any_lora else N
        pair = TWO_CTA_DECODE and M % 256 == 0 and N >= 256
        bn, splits = plan_small_m(M, Next, self.K, pair=pair)
        ws = self._ws(M, Next, x.device)
        gemm_splitk_(ws, x, self.W_ext[:Next], bn, splits, two_cta=pair)
        return ws

    def _shrink(self, x, adapter_ids):
        """``T[M, kpad] = X A_all^T`` with every row restricted to the columns of its own adapter slot."""
        from ..ops.gemm import gemm_splitk_, gemm_tn, plan_small_m, splitk_finalize
        from ..ops.paged import lora_slot_mask_

        M = x.shape[0]
        bn, splits = plan_small_m(M, self.kpad, self.K)
        if splits > 1:
            ws = self._ws(M, self.kpad, x.device)
            T = torch.empty((M, self.kpad), dtype=torch.bfloat16, device=x.device)
            gemm_splitk_(ws, x, self.A_all, bn, splits)
            return splitk_finalize(ws, T, None, None, 0, adapter_ids, 0, self.cols)
        return lora_slot_mask_(gemm_tn(x, self.A_all, bn=bn), adapter_ids, self.cols)

    def __call__(self, x, adapter_ids, any_lora: bool, residual=None, swiglu_out=None):
        from ..ops import elementwise as ew
        from ..ops.gemm import gemm_splitk_, gemm_tn, plan_small_m, splitk_finalize
        from ..ops.paged import lora_slot_mask_

        M = x.shape[0]
        if M > 512:     # prefill: compute-bound, LoRA as extra K
            if any_lora:
                T = gemm_tn(x, self.A_all, bn=64)
                lora_slot_mask_(T, adapter_ids, self.cols)
                return gemm_tn(x, self.W, a2=T, b2=self.B_all, residual=residual, swiglu_out=swiglu_out,
                               bias=None if self.bias_ext is None else self.bias_ext[:self.N])
            return gemm_tn(x, self.W, residual=residual, swiglu_out=swiglu_out,
                           bias=None if self.bias_ext is None else self.bias_ext[:self.N])
        N = self.N
        if _DECODE_PLAN == "narrow" and self.K <= NARROW_MAX_K and swiglu_out is None and 128 <= M <= 512:
            bias = None if self.bias_ext is None else self.bias_ext[:N]
            if any_lora:
                T = self._shrink(x, adapter_ids)
                return gemm_tn(x, self.W, a2=T, b2=self.B_all, residual=residual, bias=bias, bn=64, two_cta=False)
            return gemm_tn(x, self.W, residual=residual, bias=bias, bn=64, two_cta=False)
        pair = TWO_CTA_DECODE and M % 256 == 0 and N >= 256     # CTA pairs share each weight tile
        if any_lora and plan_small_m(M, N, self.K, pair=pair)[1] == 1:
            # wide projection (gate|up): the product is not split, so the low-rank update can ride in the same
            # accumulator as extra K once T = mask(X A_all^T) is known -- a skinny split-K GEMM over X alone -- and the
            # residual / SwiGLU epilogue runs in the weight-streaming GEMM itself (no [M, N] intermediate)
            T = self._shrink(x, adapter_ids)
            return gemm_tn(x, self.W, a2=T, b2=self.B_all, residual=residual, swiglu_out=swiglu_out, two_cta=pair,
                           bias=None if self.bias_ext is None else self.bias_ext[:N])
        Next = N + self.kpad if any_lora else N
        Wv = self.W_ext[:Next]
        bias = None if self.bias_ext is None else self.bias_ext[:Next]
        if _TWO_CTA_MODE == "wide":
            pair = pair and plan_small_m(M, Next, self.K, pair=True)[1] == 1
        bn, splits = plan_small_m(M, Next, self.K, pair=pair)
        y_ext = torch.empty((M, Next), dtype=torch.bfloat16, device=x.device)
        fuse_swiglu = swiglu_out is not None and not any_lora and splits == 1
        if splits > 1:
            ws = self._ws(M, Next, x.device)
            gemm_splitk_(ws, x, Wv, bn, splits, two_cta=pair)
            # the finalize pass also applies the per-row adapter-slot mask to the shrink columns
            splitk_finalize(ws, y_ext, bias, residual, N, adapter_ids if any_lora else None, N, self.cols)
        else:
            gemm_tn(x, Wv, out=y_ext, bias=bias, residual=residual, res_cols=N, bn=0 if pair else bn, two_cta=pair,
                    swiglu_out=swiglu_out if fuse_swiglu else None)
        if not any_lora:
            if swiglu_out is not None and not fuse_swiglu:
                ew.swiglu_fwd(y_ext, out=swiglu_out)
            return y_ext
        T = y_ext[:, N:]
        if splits == 1:
            lora_slot_mask_(T, adapter_ids, self.cols)
        return gemm_tn(T, self.B_all, residual=y_ext[:, :N], swiglu_out=swiglu_out)


class NativeRunner:
    def __init__(self, cfg: ModelConfig, lora_cfg: LoraConfig, kv, *, decoder=None, base: dict | None = None,
                 max_loras: int = 4, device="cuda", tp_group=None):
        """``decoder``: a trainer-side NativeDecoder whose frozen weights are shared; else ``base`` weights.

        ``tp_group``: tensor-parallel replica.  Every rank of the group runs the same engine on the same requests
        (same scheduler decisions, same seeds); this runner holds 1/T of the attention heads, of the FFN columns and
        of the vocabulary: q|k|v and gate|up are column-parallel, o and down row-parallel (partial sums all-reduced,
        the residual added on rank 0 only), the LM head is vocabulary-parallel (sampling statistics all-gathered and
        merged, so every rank draws the same token).  ``kv`` must be sized for ``num_kv_heads / T`` heads.
        The reference serves tensor-parallel models through vLLM (src/art/dev/engine.py: tensor_parallel_size)."""
        import dataclasses

        from ..ops import elementwise as ew

        self.full_cfg = cfg
        ew.rope_args(cfg, torch.device(device))     # frequency table of a scaled rotary embedding: never built under capture
        self.tp_group = tp_group
        self.tp = 1 if tp_group is None else torch.distributed.get_world_size(tp_group)
        self.tp_rank = 0 if tp_group is None else torch.distributed.get_rank(tp_group)
        T, tr = self.tp, self.tp_rank
        if T > 1:
            if decoder is not None or cfg.is_moe:
                raise ValueError("tensor-parallel runners build their own dense weight shards from `base`")
            if cfg.num_heads % T or cfg.num_kv_heads % T or cfg.intermediate_size % (16 * T) or cfg.vocab_size % (8 * T):
                raise ValueError(f"heads, FFN width and vocabulary of {cfg.name} do not divide over {T} ranks")
            cfg = dataclasses.replace(cfg, num_heads=cfg.num_heads // T, num_kv_heads=cfg.num_kv_heads // T,
                                      intermediate_size=cfg.intermediate_size // T)
        self.cfg, self.lora_cfg, self.kv, self.max_loras = cfg, lora_cfg, kv, max_loras
        self.device = torch.device(device)
        dev, bf = self.device, torch.bfloat16
        fc = self.full_cfg
        sl_q = slice(tr * cfg.q_size, (tr + 1) * cfg.q_size) if T > 1 else None
        sl_kv = slice(tr * cfg.kv_size, (tr + 1) * cfg.kv_size) if T > 1 else None
        sl_f = slice(tr * cfg.intermediate_size, (tr + 1) * cfg.intermediate_size) if T > 1 else None
        self.vocab_local = fc.vocab_size // T
        self.vocab_offset = tr * self.vocab_local
        if decoder is None:
            from ..models.native import LoraLinear  # reuse the fused-weight construction without LoRA members

            assert base is not None

            class _Shim:
                pass

            decoder = _Shim()
            decoder.embed = base["model.embed_tokens.weight"].to(dev, bf).contiguous()
            decoder.lm_head = base["lm_head.weight"][self.vocab_offset:self.vocab_offset + self.vocab_local].to(dev, bf).contiguous()
            decoder.final_norm = base["model.norm.weight"].to(dev, bf).contiguous()
            decoder.layers = []
            if cfg.is_moe:
                # the experts keep ONE adapter's factors resident (the slot loaded last), in a flat store of their own
                from ..models.moe import MoEMLP, expert_lora_order
                from ..models.native import LoraFlat
                from ..models.weights import init_lora

                zero = {k: torch.zeros_like(v) for k, v in init_lora(cfg, lora_cfg, seed=0, device=dev).items()
                        if ".mlp.experts." in k}
                self._moe_flat = LoraFlat(cfg, lora_cfg, zero, dev, order=expert_lora_order(cfg, list(zero.keys())))
            row_sl = {"self_attn.q_proj": sl_q, "self_attn.k_proj": sl_kv, "self_attn.v_proj": sl_kv,
                      "mlp.gate_proj": sl_f, "mlp.up_proj": sl_f}
            col_sl = {"self_attn.o_proj": sl_q, "mlp.down_proj": sl_f}

            def shard(name: str, t: torch.Tensor) -> torch.Tensor:
                if T == 1:
                    return t
                if name in row_sl:
                    return t[row_sl[name]]
                return t[:, col_sl[name]] if t.dim() == 2 else t

            for i in range(cfg.num_layers):
                p = f"model.layers.{i}."
                W = lambda n: shard(n, base[p + n + ".weight"]).to(dev, bf)  # noqa: E731
                wqkv = torch.cat([W("self_attn.q_proj"), W("self_attn.k_proj"), W("self_attn.v_proj")], 0)
                bqkv = (torch.cat([shard(f"self_attn.{n}", base[p + f"self_attn.{n}.bias"]).to(dev)
                                   for n in ("q_proj", "k_proj", "v_proj")]) if cfg.qkv_bias else None)
                layer = {"qkv": LoraLinear(wqkv, bqkv, [], lora_cfg.r, lora_cfg.scale, need_dgrad=False),
                         "o": LoraLinear(W("self_attn.o_proj"), None, [], lora_cfg.r, lora_cfg.scale, need_dgrad=False),
                         "ln1": base[p + "input_layernorm.weight"].to(dev, bf).contiguous(),
                         "ln2": base[p + "post_attention_layernorm.weight"].to(dev, bf).contiguous()}
                if cfg.is_moe:
                    layer["mlp"] = MoEMLP(cfg, i, base, self._moe_flat, lora_cfg, dev)
                else:
                    layer["gu"] = LoraLinear(ew.interleave_gate_up(W("mlp.gate_proj"), W("mlp.up_proj")), None, [],
                                             lora_cfg.r, lora_cfg.scale, need_dgrad=False)
                    layer["down"] = LoraLinear(W("mlp.down_proj"), None, [], lora_cfg.r, lora_cfg.scale, need_dgrad=False)
                if cfg.qk_norm:
                    layer["q_norm"] = base[p + "self_attn.q_norm.weight"].to(dev, bf).contiguous()
                    layer["k_norm"] = base[p + "self_attn.k_norm.weight"].to(dev, bf).contiguous()
                decoder.layers.append(layer)
        self.embed, self.lm_head, self.final_norm = decoder.embed, decoder.lm_head, decoder.final_norm
        q, kvw, d, F = cfg.q_size, cfg.kv_size, cfg.hidden_size, cfg.intermediate_size
        ar = lambda a, b: torch.arange(a, b, device=dev)  # noqa: E731
        fidx = torch.arange(F, device=dev)
        gate_rows = (fidx // 16) * 32 + fidx % 16
        r = lora_cfg.r
        self.layers = []
        self._ws_holder: dict = {}
        self._moe_flat = getattr(self, "_moe_flat", None)   # None: dense, or experts that read a trainer's master buffer
        self._moe_slot: int | None = None                   # adapter slot whose expert factors are resident
        self._moe_mixed = False                             # the batch at hand mixes base-model rows and adapter rows
        for i, L in enumerate(decoder.layers):
            if "gu" not in L and hasattr(L.get("mlp"), "Wg"):
                # sparse feed-forward (router + grouped experts): served through the trainer-side module, forward only
                self.layers.append({
                    "qkv": EngineLinear(L["qkv"], [("self_attn.q_proj", ar(0, q), sl_q, None),
                                                   ("self_attn.k_proj", ar(q, q + kvw), sl_kv, None),
                                                   ("self_attn.v_proj", ar(q + kvw, q + 2 * kvw), sl_kv, None)],
                                        r, max_loras, self._ws_holder),
                    "o": EngineLinear(L["o"], [("self_attn.o_proj", ar(0, d), None, sl_q)], r, max_loras, self._ws_holder),
                    "moe": L["mlp"], "ln1": L["ln1"], "ln2": L["ln2"], "q_norm": L.get("q_norm"), "k_norm": L.get("k_norm"),
                })
                continue
            if "gu" not in L:       # a trainer-side decoder keeps its feed-forward linears inside an MLP object
                mlp = L["mlp"]
                L = {**L, "gu": mlp.gu, "down": mlp.down}
            self.layers.append({
                "qkv": EngineLinear(L["qkv"], [("self_attn.q_proj", ar(0, q), sl_q, None),
                                               ("self_attn.k_proj", ar(q, q + kvw), sl_kv, None),
                                               ("self_attn.v_proj", ar(q + kvw, q + 2 * kvw), sl_kv, None)],
                                    r, max_loras, self._ws_holder),
                "o": EngineLinear(L["o"], [("self_attn.o_proj", ar(0, d), None, sl_q)], r, max_loras, self._ws_holder),
                "gu": EngineLinear(L["gu"], [("mlp.gate_proj", gate_rows, sl_f, None),
                                             ("mlp.up_proj", gate_rows + 16, sl_f, None)], r, max_loras, self._ws_holder),
                "down": EngineLinear(L["down"], [("mlp.down_proj", ar(0, d), None, sl_f)], r, max_loras, self._ws_holder),
                "ln1": L["ln1"], "ln2": L["ln2"], "q_norm": L.get("q_norm"), "k_norm": L.get("k_norm"),
            })
        self.slot_loaded = [False] * max_loras
        self.table_width: int | None = None    # fixed block-table width (else grown by doubling, which adds graph keys)

    def close(self) -> None:
        """Drop the captured decode graphs and their buffers.  A tensor-parallel runner must be closed before its
        process group is destroyed: NCCL does not finish tearing down a communicator while CUDA graphs that captured
        its collectives are alive."""
        self.drop_graphs()

    def drop_graphs(self) -> None:
        """Forget every captured decode graph (and its buffers); the next decode of each shape runs eagerly and is
        captured again.  Needed whenever an address baked into the graphs changes, e.g. a KV cache that was freed and
        re-allocated around a training step."""
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        if hasattr(self, "_dgraphs"):
            self._dgraphs.clear()
            self._dstate.clear()
            self._dseen.clear()

    # -- tensor parallel ------------------------------------------------------------------------
    def _reduce(self, x: torch.Tensor) -> torch.Tensor:
        """Sum the row-parallel partial products over the replica (in place; a no-op on one GPU)."""
        if self.tp > 1:
            torch.distributed.all_reduce(x, group=self.tp_group)
        return x

    def _res(self, x: torch.Tensor):
        """The residual enters a row-parallel projection on one rank only: the all-reduce then adds it once."""
        return x if self.tp_rank == 0 else None

    def _sample(self, hidden, inv_t, seeds, restricted: bool, top_k=None, top_p=None, min_p=None, procs=None):
        """``procs``: per-row ``(LogitProc, tokens)`` or None entries; any entry sends the step through fp32 logits
        (one GEMM), the sparse logit-edit kernel, the restricted sampler and, if asked, the top-logprobs kernel."""
        from ..ops import paged

        self._step_top = None
        if procs is not None and any(p is not None for p in procs):
            from ..ops.gemm import gemm_tn

            logits = gemm_tn(hidden, self.lm_head, out_dtype=torch.float32)
            if self.tp > 1:
                allv = torch.empty((self.tp,) + tuple(logits.shape), dtype=logits.dtype, device=logits.device)
                torch.distributed.all_gather_into_tensor(allv, logits, group=self.tp_group)
                logits = allv.permute(1, 0, 2).reshape(logits.shape[0], -1).contiguous()
            n = len(procs)
            paged.logit_adjust_(logits, paged.build_logit_edits([p if p is not None and p[0].edits else None for p in procs]))
            grammars = [p[0].grammar if p is not None else None for p in procs]
            if any(g is not None for g in grammars):
                apply_token_mask(logits, grammars + [None] * (logits.shape[0] - len(grammars)))
            kmax = max((p[0].top_logprobs for p in procs if p is not None), default=0)
            if kmax > 0:
                ti, tl = paged.top_logprobs(logits, inv_t, kmax)
                ti, tl = ti[:n].tolist(), tl[:n].tolist()
                self._step_top = [None if p is None or p[0].top_logprobs <= 0 else
                                  list(zip(ti[i][:p[0].top_logprobs], tl[i][:p[0].top_logprobs])) for i, p in enumerate(procs)]
            return paged.sample_from_logits(logits, inv_t, seeds, top_k, top_p, min_p)
        if self.tp == 1:
            if restricted:
                return paged.sample_restricted(hidden, self.lm_head, inv_t, seeds, top_k, top_p, min_p)
            return paged.sample(hidden, self.lm_head, inv_t, seeds)
        dist = torch.distributed
        if restricted:
            from ..ops.gemm import gemm_tn

            local = gemm_tn(hidden, self.lm_head, out_dtype=torch.float32)          # [M, V / T]
            allv = torch.empty((self.tp,) + tuple(local.shape), dtype=local.dtype, device=local.device)
            dist.all_gather_into_tensor(allv, local, group=self.tp_group)
            logits = allv.permute(1, 0, 2).reshape(local.shape[0], -1).contiguous()
            return paged.sample_from_logits(logits, inv_t, seeds, top_k, top_p, min_p)
        part = paged.sample_partials(hidden, self.lm_head, inv_t, seeds, self.vocab_offset)    # [splits, M, 8]
        allp = torch.empty((self.tp * part.shape[0],) + tuple(part.shape[1:]), dtype=part.dtype, device=part.device)
        dist.all_gather_into_tensor(allp, part, group=self.tp_group)
        return paged.sample_merge(allp)

    # -- adapters -----------------------------------------------------------------------------
    def set_adapter(self, slot: int, state: dict[str, torch.Tensor] | None) -> None:
        """In-device hand-off: copy (and re-lay-out) LoRA factors into adapter slot ``slot``.

        ``state`` tensors may be views of the trainer's flat fp32 master buffer; nothing touches
        the host or the disk.  The engine must be between steps (callers pause it first).
        """
        for i, L in enumerate(self.layers):
            for k in ("qkv", "o", "gu", "down"):
                if k in L:
                    L[k].load_slot(slot, i, state, self.lora_cfg.scale)
        if self._moe_flat is not None:
            # Expert factors: one adapter at a time.  Rollouts of a training run all use the newest adapter, so the
            # slot loaded last owns the experts; loading expert factors into a second slot while another slot's are
            # resident would silently serve the wrong experts to the first, so it is refused.
            has_experts = state is not None and any(".mlp.experts." in k for k in state)
            if has_experts and self._moe_slot not in (None, slot) and self.slot_loaded[self._moe_slot]:
                raise ValueError("a sparse model keeps the expert factors of one adapter resident; "
                                 f"slot {self._moe_slot} holds them (remove that adapter first, or serve with max_loras=1)")
            if has_experts or self._moe_slot == slot:
                for k, v in self._moe_flat.views.items():
                    if has_experts and k in state:
                        v.copy_(state[k])
                    else:
                        v.zero_()
                for L in self.layers:
                    if "moe" in L:
                        for lin in L["moe"].linears():
                            lin.refresh()
                self._moe_slot = slot if has_experts else None
        self.slot_loaded[slot] = state is not None

    # -- shared layer body ----------------------------------------------------------------------
    def _mlp(self, L, x2, adapter_ids, any_lora):
        from ..ops import elementwise as ew

        h2, _ = ew.rmsnorm_fwd(x2, L["ln2"], self.cfg.rms_norm_eps, want_rstd=False)
        if "moe" in L:
            moe = L["moe"]
            if not any_lora:
                return moe.forward(h2, x2, False, False)[0]
            y = moe.forward(h2, x2, True, False)[0]
            if self._moe_mixed:      # rows of the base model in the same batch: their experts run without the factors
                y0 = moe.forward(h2, x2, False, False)[0]
                y = torch.where((adapter_ids >= 0).unsqueeze(1), y, y0)
            return y
        hact = torch.empty((x2.shape[0], self.cfg.intermediate_size), dtype=x2.dtype, device=x2.device)
        L["gu"](h2, adapter_ids, any_lora, swiglu_out=hact)
        return self._reduce(L["down"](hact, adapter_ids, any_lora, residual=self._res(x2)))

    def _qkv(self, L, x, pos, adapter_ids, any_lora):
        from ..ops import elementwise as ew

        cfg = self.cfg
        h1, _ = ew.rmsnorm_fwd(x, L["ln1"], cfg.rms_norm_eps, want_rstd=False)
        qkv = L["qkv"](h1, adapter_ids, any_lora)
        if cfg.qk_norm:
            ew.headnorm_fwd_(qkv, L["q_norm"], 0, cfg.num_heads, cfg.head_dim, cfg.rms_norm_eps)
            ew.headnorm_fwd_(qkv, L["k_norm"], cfg.q_size, cfg.num_kv_heads, cfg.head_dim, cfg.rms_norm_eps)
        ew.rope_(qkv, pos, 0, cfg.num_heads + cfg.num_kv_heads, cfg.head_dim, cfg.rope_theta, **ew.rope_args(cfg, qkv.device))
        return qkv

    # -- prefill ------------------------------------------------------------------------------------
    def _prompt_forward(self, seqs: list[SeqView], write_kv: bool = True):
        """Run the decoder over the not-yet-cached tokens of ``seqs``; returns the residual stream
        ``x`` [M_new, d] and, per sequence, the row range of its new tokens."""
        from ..ops import attention as attn_ops
        from ..ops import elementwise as ew
        from ..ops import paged

        cfg, dev, bs = self.cfg, self.device, self.kv.shape[1]
        row_ranges = []
        tok, pos, gid, adapter, slot, new_rows, last_rows = [], [], [], [], [], [], []
        cached_spans = []   # (att_row_start, n_cached, blocks)
        att = 0
        for i, s in enumerate(seqs):
            n = len(s.tokens) if s.upto is None else min(s.upto, len(s.tokens))
            nc = s.num_cached
            if nc:
                cached_spans.append((att, nc, s.blocks))
                gid += [i] * nc
                att += nc
            r0 = len(tok)
            for t in range(nc, n):
                tok.append(s.tokens[t])
                pos.append(t)
                adapter.append(s.adapter)
                slot.append(s.blocks[t // bs] * bs + t % bs if write_kv else -1)
                new_rows.append(att)
                gid.append(i)
                att += 1
            row_ranges.append((r0, len(tok)))
            last_rows.append(len(tok) - 1)
        M = len(tok)
        S_att = (att + 63) // 64 * 64
        gid += [-(j + 1) for j in range(S_att - att)]
        any_lora = any(a >= 0 for a in adapter)
        self._moe_mixed = any_lora and any(a < 0 for a in adapter)
        use_index = bool(cached_spans) or S_att != M
        t_tok = torch.tensor(tok, dtype=torch.int64, device=dev)
        t_pos = torch.tensor(pos, dtype=torch.int32, device=dev)
        t_ad = torch.tensor(adapter, dtype=torch.int32, device=dev)
        t_slot = torch.tensor(slot, dtype=torch.int32, device=dev)
        t_gid = torch.tensor(gid, dtype=torch.int32, device=dev)
        t_rows = torch.tensor(new_rows, dtype=torch.int64, device=dev)
        plan = attn_ops.make_plan(t_gid, t_gid, S_att, "native")
        Hq, Hkv, hd = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        x = ew.gather_rows(self.embed, t_tok)
        span_tables = [(a0, nc, torch.tensor(bl, dtype=torch.int32, device=dev)) for a0, nc, bl in cached_spans]
        for li, L in enumerate(self.layers):
            qkv = self._qkv(L, x, t_pos, t_ad, any_lora)
            paged.kv_write(qkv, cfg.q_size, cfg.q_size + cfg.kv_size, t_slot, self.kv.k[li], self.kv.v[li])
            if use_index:
                buf = torch.zeros((S_att, qkv.shape[1]), dtype=qkv.dtype, device=dev)
                buf.index_copy_(0, t_rows, qkv)
                for a0, nc, bt in span_tables:
                    paged.kv_gather(self.kv.k[li], self.kv.v[li], bt, bs, nc, buf[a0:], cfg.q_size, cfg.q_size + cfg.kv_size)
                o_all, _ = attn_ops.forward(buf, Hq, Hkv, hd, plan, need_grad=False)
                o = o_all.index_select(0, t_rows)
            else:
                o, _ = attn_ops.forward(qkv, Hq, Hkv, hd, plan, need_grad=False)
            x2 = self._reduce(L["o"](o, t_ad, any_lora, residual=self._res(x)))
            x = self._mlp(L, x2, t_ad, any_lora)
        return x, row_ranges

    def prefill(self, seqs: list[SeqView]) -> tuple[list[int], list[float]]:
        from ..ops import elementwise as ew
        from ..ops import paged

        cfg, dev = self.cfg, self.device
        x, ranges = self._prompt_forward(seqs, write_kv=True)
        if any(s.partial for s in seqs):
            # chunks that do not reach the end of their prompt only fill the cache; sample for the others
            done = [i for i, s in enumerate(seqs) if not s.partial]
            toks: list = [None] * len(seqs)
            lps: list = [None] * len(seqs)
            self.last_top_logprobs = None
            if done:
                t, lp, tops = self._sample_rows(x, [ranges[i] for i in done], [seqs[i] for i in done])
                for j, i in enumerate(done):
                    toks[i], lps[i] = t[j], lp[j]
                if tops is not None:
                    full = [None] * len(seqs)
                    for j, i in enumerate(done):
                        full[i] = tops[j]
                    self.last_top_logprobs = [full]
            return toks, lps
        t, lp, tops = self._sample_rows(x, ranges, seqs)
        self.last_top_logprobs = [tops] if tops is not None else None
        return t, lp

    def _sample_rows(self, x, ranges, seqs):
        """Sample the next token of every sequence from the last row of its range in ``x``."""
        from ..ops import elementwise as ew

        cfg, dev = self.cfg, self.device
        t_last = torch.tensor([r1 - 1 for _, r1 in ranges], dtype=torch.int64, device=dev)
        hl = ew.gather_rows(x, t_last)
        hidden, _ = ew.rmsnorm_fwd(hl, self.final_norm, cfg.rms_norm_eps, want_rstd=False)
        inv_t = torch.tensor([0.0 if s.temperature <= 0 else 1.0 / s.temperature for s in seqs], dtype=torch.float32, device=dev)
        seeds = torch.tensor([_mix_seed(s.seed, s.step) for s in seqs], dtype=torch.int64, device=dev).to(torch.int32)
        procs = [(s.proc, s.tokens) if s.proc is not None else None for s in seqs]
        if any(s.restricted or s.proc is not None for s in seqs):
            tk = torch.tensor([s.top_k for s in seqs], dtype=torch.int32, device=dev)
            tp = torch.tensor([s.top_p for s in seqs], dtype=torch.float32, device=dev)
            mp = torch.tensor([s.min_p for s in seqs], dtype=torch.float32, device=dev)
            t, lp = self._sample(hidden, inv_t, seeds, True, tk, tp, mp, procs=procs)
        else:
            t, lp = self._sample(hidden, inv_t, seeds, False)
        return t.tolist(), lp.tolist(), self._step_top

    def score(self, tokens: list[int], n_prompt: int, adapter: int) -> list[float]:
        """Log-probabilities of ``tokens[n_prompt:]`` given what precedes them (no KV is written)."""
        from ..ops import elementwise as ew
        from ..ops import logprob_loss as lpl

        sv = SeqView(tokens, 0, [], adapter, 0.0, 0, 0)
        x, _ = self._prompt_forward([sv], write_kv=False)
        rows = torch.arange(n_prompt - 1, len(tokens) - 1, dtype=torch.int64, device=self.device)
        h, _ = ew.rmsnorm_fwd(ew.gather_rows(x, rows), self.final_norm, self.cfg.rms_norm_eps, want_rstd=False)
        tgt = torch.tensor(tokens[n_prompt:], dtype=torch.int32, device=self.device)
        if self.tp > 1:      # rare path: gather the vocabulary shards of the logits and score in PyTorch
            from ..ops.gemm import gemm_tn

            local = gemm_tn(h, self.lm_head, out_dtype=torch.float32)
            allv = torch.empty((self.tp,) + tuple(local.shape), dtype=local.dtype, device=local.device)
            torch.distributed.all_gather_into_tensor(allv, local, group=self.tp_group)
            lp = torch.log_softmax(allv.permute(1, 0, 2).reshape(local.shape[0], -1), -1)
            return lp.gather(-1, tgt.long().unsqueeze(-1)).squeeze(-1).tolist()
        part, _ = lpl.partials(h, self.lm_head, tgt)
        return lpl.grpo_tokens(part).logprobs.tolist()

    # -- decode -------------------------------------------------------------------------------------
    # The multi-step decode runs on persistent device buffers (one set per batch-size bucket) so that
    # the whole run of n_steps x (all layers + sampler + state advance) can be captured in a CUDA
    # graph and replayed: a decode step is ~500 small launches, which the host cannot issue as fast
    # as the GPU retires them.  The first use of a (bucket, n_steps, lora, splits, table width) key
    # runs eagerly, the second captures, later ones replay.
    BUCKETS = (8, 16, 32, 64, 128, 256, 512, 1024)

    def _decode_state(self, nb: int, max_blocks: int, n_steps: int):
        key = (nb, max_blocks, n_steps)
        st = self._dstate.get(key) if hasattr(self, "_dstate") else None
        if st is None:
            if not hasattr(self, "_dstate"):
                self._dstate, self._dgraphs, self._dseen = {}, {}, set()
            dev, cfg = self.device, self.cfg
            st = {
                "tokens": torch.zeros(nb, dtype=torch.int64, device=dev), "pos": torch.zeros(nb, dtype=torch.int32, device=dev),
                "ctx": torch.zeros(nb, dtype=torch.int32, device=dev), "slot": torch.full((nb,), -1, dtype=torch.int32, device=dev),
                "ad": torch.full((nb,), -1, dtype=torch.int32, device=dev), "active": torch.zeros(nb, dtype=torch.int32, device=dev),
                "inv_t": torch.zeros(nb, dtype=torch.float32, device=dev),
                "top_k": torch.zeros(nb, dtype=torch.int32, device=dev), "top_p": torch.ones(nb, dtype=torch.float32, device=dev),
                "min_p": torch.zeros(nb, dtype=torch.float32, device=dev),
                "seeds": torch.zeros((n_steps, nb), dtype=torch.int32, device=dev),
                "bt": torch.zeros((nb, max_blocks), dtype=torch.int32, device=dev),
                "out_t": torch.zeros((n_steps, nb), dtype=torch.int32, device=dev),
                "out_l": torch.zeros((n_steps, nb), dtype=torch.float32, device=dev),
                "attn_out": torch.zeros((nb, cfg.q_size), dtype=torch.bfloat16, device=dev),
                "q": torch.zeros((nb, cfg.q_size), dtype=torch.bfloat16, device=dev),
            }
            self._dstate[key] = st
        return st

    def _decode_body(self, st, n_steps: int, any_lora: bool, splits: int, ws, restricted: bool = False, procs=None):
        from ..ops import elementwise as ew
        from ..ops import paged

        prev_pdl = paged.set_pdl(os.environ.get("ARTB_PDL", "1") != "0")
        try:
            self._decode_steps(st, n_steps, any_lora, splits, ws, restricted, procs)
        finally:
            paged.set_pdl(prev_pdl)

    def _decode_steps(self, st, n_steps: int, any_lora: bool, splits: int, ws, restricted: bool, procs) -> None:
        from ..ops import elementwise as ew
        from ..ops import paged

        cfg, bs = self.cfg, self.kv.shape[1]
        Hq, Hkv, hd = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        fused = self._fused_decode_ok(st["tokens"].shape[0])
        for k in range(n_steps):
            x = ew.gather_rows(self.embed, st["tokens"])
            if fused:
                # every split projection stays in the fp32 workspace until ONE kernel finishes it together with what
                # follows it (RoPE + cache write, or the residual add + the next RMSNorm)
                h, _ = ew.rmsnorm_fwd(x, self.layers[0]["ln1"], cfg.rms_norm_eps, want_rstd=False)
                for li, L in enumerate(self.layers):
                    nxt = self.layers[li + 1]["ln1"] if li + 1 < len(self.layers) else self.final_norm
                    x, h = self._layer_decode_fused(li, L, x, h, nxt, st, any_lora, splits, ws)
                hidden = h
            else:
                for li, L in enumerate(self.layers):
                    qkv = self._qkv(L, x, st["pos"], st["ad"], any_lora)
                    paged.kv_write(qkv, cfg.q_size, cfg.q_size + cfg.kv_size, st["slot"], self.kv.k[li], self.kv.v[li])
                    paged.paged_decode(qkv, self.kv.k[li], self.kv.v[li], st["bt"], st["ctx"], Hq, Hkv, hd, st["attn_out"], splits, ws)
                    x2 = self._reduce(L["o"](st["attn_out"], st["ad"], any_lora, residual=self._res(x)))
                    x = self._mlp(L, x2, st["ad"], any_lora)
                hidden, _ = ew.rmsnorm_fwd(x, self.final_norm, cfg.rms_norm_eps, want_rstd=False)
            t, lp = self._sample(hidden, st["inv_t"], st["seeds"][k], restricted, st["top_k"], st["top_p"], st["min_p"],
                                 procs=procs)
            st["out_t"][k].copy_(t)
            st["out_l"][k].copy_(lp)
            if k + 1 < n_steps:
                paged.decode_advance(t, st["tokens"], st["pos"], st["ctx"], st["slot"], st["bt"], bs, st["active"])

    def _fused_decode_ok(self, M: int) -> bool:
        """The fused finish kernels cover one GPU per replica (a tensor-parallel replica all-reduces between the
        projection and the norm), no per-head q/k norm, the unscaled rotary embedding, dense MLPs, and adapter slots
        of at most 64 shrink columns."""
        if (self.tp > 1 or self.cfg.qk_norm or self.cfg.rope_scaling is not None or M > 512
                or os.environ.get("ARTB_DECODE_FUSED", "1") == "0"):
            return False
        L = self.layers[0]
        return all(isinstance(L.get(k), EngineLinear) and L[k].cols <= 64 for k in ("qkv", "o", "gu", "down"))

    def _layer_decode_fused(self, li: int, L, x, h, next_norm, st, any_lora: bool, splits: int, ws):
        from ..ops import paged

        cfg = self.cfg
        M, d = x.shape
        Hq, Hkv, hd = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        ad = st["ad"] if any_lora else None
        lin = L["qkv"]
        w = lin.partial_sums(h, any_lora)
        paged.decode_finalize_qkv(w, M, Hq, Hkv, hd, lin.kpad, st["pos"], cfg.rope_theta, st["slot"], self.kv.k[li],
                                  self.kv.v[li], st["q"], bias=None if lin.bias_ext is None else lin.bias_ext[:lin.N],
                                  adapter=ad, B_all=lin.B_T, cols=lin.cols)
        paged.paged_decode(st["q"], self.kv.k[li], self.kv.v[li], st["bt"], st["ctx"], Hq, Hkv, hd, st["attn_out"], splits, ws)
        lin = L["o"]
        w = lin.partial_sums(st["attn_out"], any_lora)
        x2, h2 = torch.empty_like(x), torch.empty_like(x)
        paged.decode_finalize_norm(w, M, d, lin.kpad, x2, bias=None if lin.bias_ext is None else lin.bias_ext[:d],
                                   residual=x, adapter=ad, B_all=lin.B_T, cols=lin.cols, norm_w=L["ln2"],
                                   eps=cfg.rms_norm_eps, h_out=h2)
        hact = torch.empty((M, cfg.intermediate_size), dtype=x.dtype, device=x.device)
        L["gu"](h2, st["ad"], any_lora, swiglu_out=hact)
        lin = L["down"]
        w = lin.partial_sums(hact, any_lora)
        x3, h3 = torch.empty_like(x), torch.empty_like(x)
        paged.decode_finalize_norm(w, M, d, lin.kpad, x3, bias=None if lin.bias_ext is None else lin.bias_ext[:d],
                                   residual=x2, adapter=ad, B_all=lin.B_T, cols=lin.cols, norm_w=next_norm,
                                   eps=cfg.rms_norm_eps, h_out=h3)
        return x3, h3

    def decode(self, seqs: list[SeqView], n_steps: int, use_graph: bool = True) -> tuple[list[list[int]], list[list[float]]]:
        cfg, dev, bs = self.cfg, self.device, self.kv.shape[1]
        n = len(seqs)
        nb = next((b for b in self.BUCKETS if b >= n), (n + 255) // 256 * 256)
        need_blocks = max(len(s.blocks) for s in seqs)
        max_blocks = self.table_width or 64
        while max_blocks < need_blocks:
            max_blocks *= 2
        st = self._decode_state(nb, max_blocks, n_steps)
        import numpy as np

        lens = [len(s.tokens) for s in seqs]
        pad = nb - n
        # host-side staging with numpy: one array per input instead of one small tensor per sequence
        bt = np.zeros((nb, max_blocks), dtype=np.int32)
        for i, s in enumerate(seqs):
            bt[i, :len(s.blocks)] = s.blocks
        la = np.zeros(nb, dtype=np.int64)
        la[:n] = lens
        last = np.zeros(nb, dtype=np.int64)
        last[:n] = [s.tokens[-1] for s in seqs]
        slot = np.full(nb, -1, dtype=np.int32)
        rows = np.arange(n)
        slot[:n] = bt[rows, (la[:n] - 1) // bs] * bs + (la[:n] - 1) % bs
        ad = np.full(nb, -1, dtype=np.int32)
        ad[:n] = [s.adapter for s in seqs]
        act = np.zeros(nb, dtype=np.int32)
        act[:n] = 1
        inv_t = np.zeros(nb, dtype=np.float32)
        inv_t[:n] = [0.0 if s.temperature <= 0 else 1.0 / s.temperature for s in seqs]
        # _mix_seed(seed, step + k) for every sequence and step, in 64-bit arithmetic
        sd = np.zeros((1, nb), dtype=np.uint64)
        sd[0, :n] = [s.seed & 0xFFFFFFFF for s in seqs]
        stp = np.zeros((1, nb), dtype=np.uint64)
        stp[0, :n] = [s.step for s in seqs]
        ks = np.arange(n_steps, dtype=np.uint64)[:, None]
        seeds = (sd * np.uint64(0x9E3779B1) + (stp + ks) * np.uint64(0x85EBCA77) + np.uint64(0x165667B1)) & np.uint64(0xFFFFFFFF)
        seeds[:, n:] = 0
        st["bt"].copy_(torch.from_numpy(bt), non_blocking=True)
        st["tokens"].copy_(torch.from_numpy(last), non_blocking=True)
        st["pos"].copy_(torch.from_numpy((la - 1).clip(min=0).astype(np.int32)), non_blocking=True)
        st["ctx"].copy_(torch.from_numpy(la.astype(np.int32)), non_blocking=True)
        st["slot"].copy_(torch.from_numpy(slot), non_blocking=True)
        st["ad"].copy_(torch.from_numpy(ad), non_blocking=True)
        st["active"].copy_(torch.from_numpy(act), non_blocking=True)
        st["inv_t"].copy_(torch.from_numpy(inv_t), non_blocking=True)
        st["seeds"].copy_(torch.from_numpy(seeds.astype(np.int64)).to(torch.int32), non_blocking=True)
        any_lora = any(s.adapter >= 0 for s in seqs)
        self._moe_mixed = any_lora and (pad > 0 or any(s.adapter < 0 for s in seqs))
        procs = None
        if any(s.proc is not None for s in seqs):
            # logit edits depend on every token sampled so far: one step at a time, outside the captured graphs
            if n_steps != 1:
                raise ValueError("sequences with penalties, logit_bias or top_logprobs decode one step per call")
            procs = [(s.proc, s.tokens) if s.proc is not None else None for s in seqs] + [None] * pad
            use_graph = False
        restricted = any(s.restricted for s in seqs) or procs is not None
        if restricted:
            st["top_k"].copy_(torch.tensor([s.top_k for s in seqs] + [0] * pad, dtype=torch.int32), non_blocking=True)
            st["top_p"].copy_(torch.tensor([s.top_p for s in seqs] + [1.0] * pad, dtype=torch.float32), non_blocking=True)
            st["min_p"].copy_(torch.tensor([s.min_p for s in seqs] + [0.0] * pad, dtype=torch.float32), non_blocking=True)
        max_ctx = max(lens) + n_steps
        splits = 1 if nb * cfg.num_kv_heads >= 128 else min(8, max(1, 1 << (max(1, max_ctx // 512).bit_length() - 1)))
        key = (nb, max_blocks, n_steps, any_lora, splits, restricted, self._moe_mixed)
        ws = None
        if splits > 1:
            ws = st.get(("ws", splits))
            if ws is None:
                ws = st[("ws", splits)] = torch.empty(nb * cfg.num_heads * splits * (cfg.head_dim + 2), dtype=torch.float32, device=dev)
        graph = self._dgraphs.get(key) if procs is None else None
        self.last_top_logprobs = None
        if procs is not None:
            self._decode_body(st, 1, any_lora, splits, ws, True, procs=procs)
            self.last_top_logprobs = [self._step_top] if self._step_top is not None else None
        elif graph is not None:
            graph.replay()
        elif use_graph and key in self._dseen and not os.environ.get("ARTB_DECODE_NO_GRAPH"):
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                self._decode_body(st, n_steps, any_lora, splits, ws, restricted)
            self._dgraphs[key] = graph
            graph.replay()
        else:
            self._dseen.add(key)
            self._decode_body(st, n_steps, any_lora, splits, ws, restricted)
        out_t = st["out_t"][:, :n].tolist()
        out_l = st["out_l"][:, :n].tolist()
        return out_t, out_l
