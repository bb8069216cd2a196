"""Front-ends for the rollout-engine kernels: KV-cache write/gather, paged decode attention,
multi-LoRA slot mask, fused LM-head sampler, top-k / top-p sampler, device-side decode bookkeeping."""
from __future__ import annotations

import ctypes

import torch

from . import _lib

vp, ci, cl = ctypes.c_void_p, ctypes.c_int, ctypes.c_long
_sigs = {
    "artb_kv_write": [vp, ci, ci, ci, vp, vp, vp, ci, ci, cl, vp, vp],
    "artb_kv_gather": [vp, vp, vp, ci, ci, vp, ci, ci, ci, ci, cl, vp, vp],
    "artb_paged_decode": [vp, ci, vp, vp, vp, ci, vp, ci, ci, ci, ci, ci, vp, ci, vp, ci, cl, vp, vp],
    "artb_lora_slot_mask": [vp, ci, vp, cl, ci, ci, vp, vp],
    "artb_decode_advance": [vp, vp, vp, vp, vp, vp, ci, ci, vp, ci, vp],
    "artb_sample_partials": [vp, ci, vp, ci, vp, vp, vp, ci, ci, ci, ci, ci, vp, vp],
    "artb_sample_merge": [vp, ci, ci, vp, vp, vp],
    "artb_logprob_splits": [ci, ci],
    "artb_sample_restricted": [vp, cl, vp, vp, vp, vp, vp, ci, ci, ci, vp, vp, vp],
    "artb_logit_adjust": [vp, cl, vp, vp, vp, vp, vp, ci, ci, ci, vp],
    "artb_top_logprobs": [vp, cl, vp, ci, ci, ci, vp, vp, vp],
    "artb_set_pdl": [ci],
    "artb_decode_finalize_norm": [vp, ci, ci, ci, ci, vp, vp, ci, vp, vp, ci, ci, vp, ctypes.c_float, vp, ci, vp, ci, vp],
    "artb_decode_finalize_qkv": [vp, ci, ci, ci, ci, ci, ci, vp, vp, vp, ci, ci, vp, ctypes.c_float, vp, vp, vp, vp, ci, cl, vp,
                                 vp],
}
_bound: dict[str, object] = {}


def _f(name: str):
    fn = _bound.get(name)
    if fn is None:
        fn = getattr(_lib.kernels(), name)
        fn.argtypes = _sigs[name]
        fn.restype = ci
        _bound[name] = fn
    return fn


def _cache_slots(cache: torch.Tensor) -> int:
    """Token slots of a paged cache [blocks, block_size, heads, head_dim] (what a checked build compares slots with)."""
    return cache.shape[0] * cache.shape[1]


def kv_write(qkv: torch.Tensor, k_col: int, v_col: int, slot: torch.Tensor, k_cache: torch.Tensor,
             v_cache: torch.Tensor) -> None:
    kv_width = k_cache.shape[-2] * k_cache.shape[-1]
    _lib.check_rc(_f("artb_kv_write")(_lib.ptr(qkv), qkv.stride(0), k_col, v_col, _lib.ptr(slot), _lib.ptr(k_cache),
                                      _lib.ptr(v_cache), qkv.shape[0], kv_width, _cache_slots(k_cache),
                                      _lib.ptr(_lib.status_word(qkv.device)), _lib.stream_ptr()), "kv_write")


def set_pdl(on: bool) -> bool:
    """Programmatic dependent launch for the decode-step kernels launched from now on (returns the previous setting):
    each may start its prologue while its predecessor in the stream drains, and waits on the device before touching
    global memory."""
    return bool(_f("artb_set_pdl")(1 if on else 0))


def decode_finalize_norm(ws: torch.Tensor, M: int, N: int, kpad: int, x_out: torch.Tensor, *, bias: torch.Tensor | None = None,
                         residual: torch.Tensor | None = None, adapter: torch.Tensor | None = None,
                         B_all: torch.Tensor | None = None, cols: int = 0, norm_w: torch.Tensor | None = None,
                         eps: float = 1e-6, h_out: torch.Tensor | None = None) -> None:
    """Finish a decode-time split-K projection whose fp32 partial sums sit in ``ws[:M, :N]`` (and, with ``adapter``, the
    stacked LoRA shrink products in ``ws[:M, N:N+kpad]``; ``B_all`` is the scaled LoRA B transposed, [kpad, N]):
    ``x_out = bf16(ws + bias + residual + T_slot sB_slot^T)``
    and, with ``norm_w``, ``h_out = RMSNorm(x_out) * norm_w``.  The consumed workspace columns are left zero."""
    _lib.check_rc(_f("artb_decode_finalize_norm")(
        _lib.ptr(ws), ws.stride(0), M, N, kpad, _lib.ptr(bias), _lib.ptr(residual),
        residual.stride(0) if residual is not None else 0, _lib.ptr(adapter), _lib.ptr(B_all),
        B_all.stride(0) if B_all is not None else 0, cols, _lib.ptr(norm_w), eps, _lib.ptr(x_out), x_out.stride(0),
        _lib.ptr(h_out), h_out.stride(0) if h_out is not None else 0, _lib.stream_ptr()), "decode_finalize_norm")


def decode_finalize_qkv(ws: torch.Tensor, M: int, Hq: int, Hkv: int, hd: int, kpad: int, pos: torch.Tensor, theta: float,
                        slot: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, q_out: torch.Tensor, *,
                        bias: torch.Tensor | None = None, adapter: torch.Tensor | None = None,
                        B_all: torch.Tensor | None = None, cols: int = 0) -> None:
    """Finish the decode-time q|k|v projection from its split-K workspace: bias, LoRA expand of the row's adapter slot,
    RoPE on q and k; q goes to ``q_out`` [M, Hq*hd], k and v straight into the paged cache at ``slot``."""
    _lib.check_rc(_f("artb_decode_finalize_qkv")(
        _lib.ptr(ws), ws.stride(0), M, Hq, Hkv, hd, kpad, _lib.ptr(bias), _lib.ptr(adapter), _lib.ptr(B_all),
        B_all.stride(0) if B_all is not None else 0, cols, _lib.ptr(pos), theta, _lib.ptr(slot), _lib.ptr(k_cache),
        _lib.ptr(v_cache), _lib.ptr(q_out), q_out.stride(0), _cache_slots(k_cache), _lib.ptr(_lib.status_word(ws.device)),
        _lib.stream_ptr()), "decode_finalize_qkv")


def kv_gather(k_cache: torch.Tensor, v_cache: torch.Tensor, block_table_row: torch.Tensor, block_size: int, n_tok: int,
              dst: torch.Tensor, k_col: int, v_col: int) -> None:
    kv_width = k_cache.shape[-2] * k_cache.shape[-1]
    _lib.check_rc(_f("artb_kv_gather")(_lib.ptr(k_cache), _lib.ptr(v_cache), _lib.ptr(block_table_row), block_size,
                                       n_tok, _lib.ptr(dst), dst.stride(0), k_col, v_col, kv_width, k_cache.shape[0],
                                       _lib.ptr(_lib.status_word(dst.device)), _lib.stream_ptr()), "kv_gather")


def paged_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                 ctx_len: torch.Tensor, Hq: int, Hkv: int, hd: int, out: torch.Tensor, splits: int = 1,
                 ws: torch.Tensor | None = None) -> torch.Tensor:
    """q [n, >=Hq*hd] (row stride arbitrary), caches [blocks, block_size, Hkv, hd]; out [n, Hq*hd]."""
    n = q.shape[0]
    block_size = k_cache.shape[1]
    if splits > 1 and ws is None:
        ws = torch.empty(n * Hq * splits * (hd + 2), dtype=torch.float32, device=q.device)
    _lib.check_rc(_f("artb_paged_decode")(_lib.ptr(q), q.stride(0), _lib.ptr(k_cache), _lib.ptr(v_cache),
                                          _lib.ptr(block_table), block_table.stride(0), _lib.ptr(ctx_len), block_size,
                                          n, Hq, Hkv, hd, _lib.ptr(out), out.stride(0), _lib.ptr(ws), splits,
                                          k_cache.shape[0], _lib.ptr(_lib.status_word(q.device)), _lib.stream_ptr()),
                  "paged_decode")
    return out


def lora_slot_mask_(T: torch.Tensor, adapter: torch.Tensor, cols_per_adapter: int) -> torch.Tensor:
    _lib.check_rc(_f("artb_lora_slot_mask")(_lib.ptr(T), T.stride(0), _lib.ptr(adapter), T.shape[0], T.shape[1],
                                            cols_per_adapter, _lib.ptr(_lib.status_word(T.device)), _lib.stream_ptr()),
                  "lora_slot_mask")
    return T


def decode_advance(sampled, tokens, pos, ctx_len, slot, block_table, block_size: int, active=None) -> None:
    _lib.check_rc(_f("artb_decode_advance")(_lib.ptr(sampled), _lib.ptr(tokens), _lib.ptr(pos), _lib.ptr(ctx_len),
                                            _lib.ptr(slot), _lib.ptr(block_table), block_table.stride(0), block_size,
                                            _lib.ptr(active), tokens.numel(), _lib.stream_ptr()), "decode_advance")


def sample_partials(hidden: torch.Tensor, lm_head: torch.Tensor, inv_temp: torch.Tensor, row_seed: torch.Tensor,
                    vocab_offset: int = 0) -> torch.Tensor:
    """Sampling statistics of one vocabulary shard: ``[splits, M, 8]`` fp32 (running max, sum of exponentials, best
    perturbed score with its index and logit).  Partials of different shards concatenate along dim 0 and
    :func:`sample_merge` reduces them, which is all a vocabulary-parallel LM head has to exchange."""
    M, K = hidden.shape
    V = lm_head.shape[0]
    splits = _f("artb_logprob_splits")(M, V)
    part = torch.empty((splits, M, 8), dtype=torch.float32, device=hidden.device)
    _lib.check_rc(_f("artb_sample_partials")(_lib.ptr(hidden), hidden.stride(0), _lib.ptr(lm_head), lm_head.stride(0),
                                             _lib.ptr(inv_temp), _lib.ptr(row_seed), _lib.ptr(part), M, V, K, splits,
                                             vocab_offset, _lib.ptr(_lib.status_word(hidden.device)),
                                             _lib.stream_ptr()), "sample_partials")
    return part


def sample_merge(part: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Reduce ``[parts, M, 8]`` sampling statistics to (token int32 [M], logprob fp32 [M])."""
    parts, M = part.shape[0], part.shape[1]
    tok = torch.empty(M, dtype=torch.int32, device=part.device)
    lp = torch.empty(M, dtype=torch.float32, device=part.device)
    _lib.check_rc(_f("artb_sample_merge")(_lib.ptr(part), parts, M, _lib.ptr(tok), _lib.ptr(lp), _lib.stream_ptr()),
                  "sample_merge")
    return tok, lp


def sample(hidden: torch.Tensor, lm_head: torch.Tensor, inv_temp: torch.Tensor, row_seed: torch.Tensor,
           vocab_offset: int = 0) -> tuple[torch.Tensor, torch.Tensor]:
    """Fused LM head + Gumbel-max sampling.  Returns (token int32 [M], logprob fp32 [M])."""
    return sample_merge(sample_partials(hidden, lm_head, inv_temp, row_seed, vocab_offset))


def sample_restricted(hidden: torch.Tensor, lm_head: torch.Tensor, inv_temp: torch.Tensor, row_seed: torch.Tensor,
                      top_k: torch.Tensor, top_p: torch.Tensor, min_p: torch.Tensor | None = None,
                      vocab_offset: int = 0) -> tuple[torch.Tensor, torch.Tensor]:
    """LM head + top-k / top-p sampling: fp32 logits from one GEMM, then one CTA per row selects the thresholds by
    radix select and samples with the same Gumbel noise as :func:`sample` (identical tokens when nothing is
    restricted).  ``top_k`` int32 [M] (<= 0: off), ``top_p`` fp32 [M] (>= 1: off), ``min_p`` fp32 [M] (<= 0: off)."""
    from .gemm import gemm_tn

    logits = gemm_tn(hidden, lm_head, out_dtype=torch.float32)
    return sample_from_logits(logits, inv_temp, row_seed, top_k, top_p, min_p, vocab_offset)


def sample_from_logits(logits: torch.Tensor, inv_temp: torch.Tensor, row_seed: torch.Tensor, top_k: torch.Tensor,
                       top_p: torch.Tensor, min_p: torch.Tensor | None = None,
                       vocab_offset: int = 0) -> tuple[torch.Tensor, torch.Tensor]:
    """The sampling half of :func:`sample_restricted` on given fp32 logits [M, V] (unit inner stride)."""
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise ValueError("logits must be fp32 with unit inner stride")
    M, V = logits.shape
    tok = torch.empty(M, dtype=torch.int32, device=logits.device)
    lp = torch.empty(M, dtype=torch.float32, device=logits.device)
    _lib.check_rc(_f("artb_sample_restricted")(_lib.ptr(logits), logits.stride(0), _lib.ptr(inv_temp), _lib.ptr(row_seed),
                                               _lib.ptr(top_k), _lib.ptr(top_p), _lib.ptr(min_p), M, V, vocab_offset,
                                               _lib.ptr(tok),
                                               _lib.ptr(lp), _lib.stream_ptr()), "sample_restricted")
    return tok, lp


def reference_restrict(logits: torch.Tensor, top_k: int, top_p: float, min_p: float = 0.0) -> torch.Tensor:
    """Boolean keep-mask of one row of (temperature-scaled) logits: min-p, then top-k, then top-p on the renormalised
    rest; values equal to a threshold are kept.  Plain PyTorch; the oracle of :func:`sample_restricted`."""
    x = logits.float()
    keep = torch.ones_like(x, dtype=torch.bool)
    if min_p > 0:
        import math

        keep &= x >= x.max() + math.log(min(min_p, 1.0))
    if 0 < top_k < x.numel():
        keep &= x >= x.topk(top_k).values[-1]
    if top_p < 1.0:
        xs = torch.where(keep, x, torch.full_like(x, float("-inf")))
        probs = torch.softmax(xs, -1)
        sp, _ = probs.sort(descending=True)
        cum = sp.cumsum(-1)
        n_keep = int((cum < top_p).sum().item()) + 1           # smallest prefix whose mass reaches top_p
        thr = sp[min(n_keep, sp.numel()) - 1]
        keep &= probs >= thr
    return keep


# ------------------------------------------------------------------------- logit processing
def build_logit_edits(per_row: list) -> tuple[list[int], list[int], list[float], list[float], list[float]] | None:
    """Sparse logit edits for a batch; ``per_row[i]`` is None or ``(proc, tokens)``: ``proc`` has
    ``repetition_penalty``, ``presence_penalty``, ``frequency_penalty``, ``logit_bias`` ({token: bias}) and ``n_prompt``;
    ``tokens`` is the sequence so far (prompt, then output).

    Semantics (those of the OpenAI API and of the sampler the reference serves through,
    ``src/art/local/vllm.py:234-247``): the repetition penalty divides positive / multiplies negative logits of every
    token that occurs in the prompt or the output; the frequency penalty subtracts ``f * count`` and the presence
    penalty ``p`` for tokens of the output; the bias is added last.  All edits of one (row, token) are merged, so
    the device kernel writes every logit at most once."""
    rows, toks, mp, mn, sub = [], [], [], [], []
    for i, item in enumerate(per_row):
        if item is None:
            continue
        a, tokens = item
        output_ids = tokens[a.n_prompt:]
        edits: dict[int, list[float]] = {}      # token -> [mul_pos, mul_neg, sub]
        rp = float(a.repetition_penalty or 1.0)
        if rp != 1.0 and rp > 0:
            for t in set(tokens):
                edits[t] = [1.0 / rp, rp, 0.0]
        fp, pp = float(a.frequency_penalty or 0.0), float(a.presence_penalty or 0.0)
        if fp or pp:
            counts: dict[int, int] = {}
            for t in output_ids:
                counts[t] = counts.get(t, 0) + 1
            for t, c in counts.items():
                edits.setdefault(t, [1.0, 1.0, 0.0])[2] += fp * c + pp
        for t, b in (a.logit_bias or {}).items():
            edits.setdefault(int(t), [1.0, 1.0, 0.0])[2] -= float(b)
        banned: set[int] = set()
        if getattr(a, "min_tokens", 0) > len(output_ids):
            banned.update(int(t) for t in getattr(a, "end_ids", ()))
        for word in getattr(a, "bad_words_ids", None) or []:
            if word and (len(word) == 1 or (len(output_ids) >= len(word) - 1 and list(output_ids[len(output_ids) - len(word) + 1:]) == list(word[:-1]))):
                banned.add(int(word[-1]))
        for t in banned:
            edits[t] = [0.0, 0.0, 1e30]          # x -> 0 * x - 1e30: out of reach of any sampler, and finite
        for t, (p_, n_, s_) in edits.items():
            rows.append(i)
            toks.append(int(t))
            mp.append(p_)
            mn.append(n_)
            sub.append(s_)
    return (rows, toks, mp, mn, sub) if rows else None


def logit_adjust_(logits: torch.Tensor, edits) -> torch.Tensor:
    """Apply :func:`build_logit_edits` output to fp32 ``logits`` [M, V] in place (CUDA kernel, or PyTorch on CPU)."""
    if edits is None:
        return logits
    rows, toks, mp, mn, sub = edits
    dev = logits.device
    if not logits.is_cuda:
        r, t = torch.tensor(rows), torch.tensor(toks)
        ok = (t >= 0) & (t < logits.shape[1])
        r, t = r[ok], t[ok]
        x = logits[r, t]
        x = torch.where(x > 0, x * torch.tensor(mp)[ok], x * torch.tensor(mn)[ok]) - torch.tensor(sub)[ok]
        logits[r, t] = x
        return logits
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise ValueError("logits must be fp32 with unit inner stride")
    ti = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)      # noqa: E731
    tf = lambda v: torch.tensor(v, dtype=torch.float32, device=dev)    # noqa: E731
    r, t, a, b, c = ti(rows), ti(toks), tf(mp), tf(mn), tf(sub)
    _lib.check_rc(_f("artb_logit_adjust")(_lib.ptr(logits), logits.stride(0), _lib.ptr(r), _lib.ptr(t), _lib.ptr(a),
                                          _lib.ptr(b), _lib.ptr(c), len(rows), logits.shape[0], logits.shape[1],
                                          _lib.stream_ptr()), "logit_adjust")
    return logits


def top_logprobs(logits: torch.Tensor, inv_temp: torch.Tensor | None, k: int) -> tuple[torch.Tensor, torch.Tensor]:
    """(token int32 [M, k], logprob fp32 [M, k]) of the k most likely tokens under ``softmax(logits * inv_temp)``
    (rows with ``inv_temp`` 0, i.e. greedy requests, are reported at temperature 1)."""
    M, V = logits.shape
    if not logits.is_cuda:
        it = torch.ones(M) if inv_temp is None else torch.where(inv_temp > 0, inv_temp, torch.ones_like(inv_temp))
        lp = torch.log_softmax(logits.float() * it[:, None], -1)
        v, i = lp.topk(min(k, V), -1)
        return i.to(torch.int32), v
    tok = torch.empty((M, k), dtype=torch.int32, device=logits.device)
    lp = torch.empty((M, k), dtype=torch.float32, device=logits.device)
    _lib.check_rc(_f("artb_top_logprobs")(_lib.ptr(logits), logits.stride(0), _lib.ptr(inv_temp), M, V, k, _lib.ptr(tok),
                                          _lib.ptr(lp), _lib.stream_ptr()), "top_logprobs")
    return tok, lp
